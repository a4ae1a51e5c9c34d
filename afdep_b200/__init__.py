"""afdep_b200 — Blackwell-native expert-parallel communication for attention-FFN disaggregation.

Public surface, the same names the reference exports (afdep/__init__.py:4-7):
``Buffer``, ``Config``, ``ReceiveResult`` and ``__version__``.  Importing the package pulls in
neither torch nor the CUDA extension; both load when the first ``Buffer`` is built.
"""

from .buffer import (
    AfdepError,
    AfdepRouteError,
    AfdepTimeoutError,
    Buffer,
    DeepEPBuffer,
    DeepEPConfig,
    DispatchHandle,
    ElasticBuffer,
    ReceiveResult,
)
from .config import Config

__version__ = "0.1.0"

__all__ = [
    "AfdepError",
    "AfdepRouteError",
    "AfdepTimeoutError",
    "Buffer",
    "Config",
    "DeepEPBuffer",
    "DeepEPConfig",
    "DispatchHandle",
    "ElasticBuffer",
    "ReceiveResult",
    "__version__",
]
