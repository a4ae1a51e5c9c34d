"""``python -m afdep doctor`` forwards to ``python -m afdep_b200 doctor``."""

from afdep_b200.__main__ import main

if __name__ == "__main__":
    main()
