"""Drop-in name for code written against the reference package: ``import afdep`` keeps
working and resolves to the Blackwell-native implementation in ``afdep_b200``."""

from afdep_b200 import *  # noqa: F401,F403
from afdep_b200 import __all__, __version__  # noqa: F401
