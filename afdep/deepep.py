"""Module path the reference uses for its role API (``afdep.deepep``)."""

from afdep_b200.buffer import *  # noqa: F401,F403
from afdep_b200.buffer import Buffer, DeepEPBuffer, DeepEPConfig, DispatchHandle, ElasticBuffer, ReceiveResult  # noqa: F401
from afdep_b200.config import *  # noqa: F401,F403
from afdep_b200.config import Config  # noqa: F401
