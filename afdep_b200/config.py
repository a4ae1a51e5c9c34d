"""Static description of one attention-FFN-disaggregated (AFD) expert-parallel exchange.

`Config` is the only thing every rank must agree on.  It carries the same fields, defaults
and validation messages as the reference's dataclass (afdep/deepep.py:36-124) so existing
callers keep working, but nothing in it depends on torch or on a GPU: the module imports in
a bare interpreter (the reference guarantees that too, tests/unit/test_deepep_build.py:55-66).

Topology convention (docs/api.md:10): ranks ``[0, ffn_ranks)`` are FFN ranks, each owning
``num_experts // ffn_ranks`` consecutive experts; the remaining ``attention_ranks`` ranks
originate every token.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Literal

MAX_RANKS = 1024
MAX_LOGICAL_EXPERTS = 2048
MAX_EXPERTS_PER_RANK = 256
MAX_TOP_K = 32
HIDDEN_ALIGNMENT = 256
FP8_GROUP_SIZE = 128
MIN_COMM_SMS = 4
# The reference reserves 24 of an H100's 132 SMs for communication (afdep/deepep.py:30);
# the same share of a 148-SM B200 is 27.
DEFAULT_COMM_SM_FRACTION = 24 / 132
INT32_MAX = (1 << 31) - 1

# One NVSwitch domain of B200s holds eight GPUs; the native transport keeps its peer table
# in kernel parameters, so this is a hard limit of the CUDA path (not of `Config`).
NATIVE_MAX_RANKS = 8

_POSITIVE = (
    "capacity_tokens_per_rank",
    "hidden_size",
    "num_experts",
    "top_k",
    "ffn_ranks",
    "attention_ranks",
    "expert_alignment",
    "cpu_timeout_s",
    "gpu_timeout_s",
)
_NONNEGATIVE = ("num_sms", "num_qps")
_BOOLEANS = ("allow_hybrid_mode", "role_aware")


def _is_int(value: object) -> bool:
    # bool is a subclass of int; the contract rejects it explicitly.
    return type(value) is int


def align_up(value: int, alignment: int) -> int:
    return (value + alignment - 1) // alignment * alignment


@dataclass(frozen=True)
class Config:
    """Expert ownership and registered capacity of one Buffer; identical on all ranks.

    ``allow_hybrid_mode``, ``num_qps`` and ``rdma_traffic_class`` describe the reference's
    RDMA scale-out transport.  They are validated and compared across ranks exactly like
    the reference does, and otherwise ignored: this library moves data over one NVLink
    domain only.
    """

    capacity_tokens_per_rank: int
    hidden_size: int
    num_experts: int
    top_k: int
    ffn_ranks: int
    attention_ranks: int
    expert_alignment: int = 128
    payload: Literal["bf16", "fp8"] = "bf16"
    allow_hybrid_mode: bool = True
    num_sms: int = 0
    num_qps: int = 0
    rdma_traffic_class: int = 0
    cpu_timeout_s: int = 120
    gpu_timeout_s: int = 120
    role_aware: bool = True
    # Not in the reference's dataclass: the form of an FP8 payload's scales.  "fp32" is the
    # reference's public contract (one fp32 scale per 128 channels).  "ue8m0x4" carries the scales
    # as exponent bytes packed four to an int32 word, the element the reference's native layer
    # also admits (deep_ep/include/deep_ep/common/compiled.cuh:74-77) and the one Blackwell's
    # block-scaled MMA consumes; the exchange moves the words untouched.
    scale_format: Literal["fp32", "ue8m0x4"] = "fp32"

    def __post_init__(self) -> None:
        for name in _POSITIVE:
            value = getattr(self, name)
            if not _is_int(value) or not 0 < value < INT32_MAX:
                raise ValueError(f"{name} must be a positive int32 integer")
        for name in _NONNEGATIVE:
            value = getattr(self, name)
            if not _is_int(value) or not 0 <= value < INT32_MAX:
                raise ValueError(f"{name} must be a nonnegative int32 integer")
        for name in _BOOLEANS:
            if type(getattr(self, name)) is not bool:
                raise ValueError(f"{name} must be a boolean")
        if not _is_int(self.rdma_traffic_class) or not 0 <= self.rdma_traffic_class <= 255:
            raise ValueError("rdma_traffic_class must be an integer in [0,255]")
        if self.hidden_size % HIDDEN_ALIGNMENT:
            raise ValueError("hidden_size must be a multiple of 256")
        if self.num_experts % self.ffn_ranks:
            raise ValueError("num_experts must divide evenly across FFN ranks")
        if self.top_k > min(MAX_TOP_K, self.num_experts):
            raise ValueError("top_k must be <=32 and <=num_experts")
        if self.payload not in ("bf16", "fp8"):
            raise ValueError("payload must be 'bf16' or 'fp8'")
        if self.scale_format not in ("fp32", "ue8m0x4"):
            raise ValueError("scale_format must be 'fp32' or 'ue8m0x4'")
        if self.scale_format != "fp32" and self.payload != "fp8":
            raise ValueError("scale_format applies to FP8 payloads only")
        if (
            self.world_size > MAX_RANKS
            or self.logical_experts > MAX_LOGICAL_EXPERTS
            or self.experts_per_rank > MAX_EXPERTS_PER_RANK
        ):
            raise ValueError("expert topology exceeds the supported workspace bounds")
        if self.receive_rows(self.capacity_tokens_per_rank) > INT32_MAX:
            raise ValueError("receive capacity exceeds int32 indexing")

    # ---- derived geometry -------------------------------------------------------------
    @property
    def world_size(self) -> int:
        return self.ffn_ranks + self.attention_ranks

    @property
    def experts_per_rank(self) -> int:
        return self.num_experts // self.ffn_ranks

    @property
    def logical_experts(self) -> int:
        """Experts counted as if attention ranks owned a block too.

        The reference needs these dummy slots for its symmetric transport
        (afdep/deepep.py:111-114).  Here roles are native and nothing is allocated for
        them; the property is kept because callers size routing tables with it.
        """
        return self.world_size * self.experts_per_rank

    @property
    def is_fp8(self) -> bool:
        return self.payload == "fp8"

    @property
    def scale_groups(self) -> int:
        """4-byte scale elements per row of an FP8 payload: one fp32 scale per 128 channels, or
        one int32 word per four of them when the scales travel as packed exponent bytes."""
        groups = self.hidden_size // FP8_GROUP_SIZE
        return (groups + 3) // 4 if self.scale_packed else groups

    @property
    def scale_packed(self) -> bool:
        return self.scale_format == "ue8m0x4"

    def receive_rows(self, bucket: int) -> int:
        """Upper bound on expert-major rows an FFN rank can receive for ``bucket``.

        Each source contributes at most ``bucket * min(top_k, experts_per_rank)`` rows and
        every expert segment may be padded by up to ``expert_alignment - 1`` rows
        (afdep/deepep.py:116-124).  ``role_aware=False`` reproduces the reference's
        generic control, where FFN ranks are counted as sources as well.
        """
        sources = self.attention_ranks if self.role_aware else self.world_size
        rows = sources * bucket * min(self.top_k, self.experts_per_rank)
        rows += (self.expert_alignment - 1) * self.experts_per_rank
        return align_up(rows, self.expert_alignment)

    def records_per_source(self, bucket: int) -> int:
        """Wire records one attention rank can send to one FFN rank: one per token."""
        return bucket

    def resolved_num_sms(self, device_sms: int) -> int:
        """Communication CTAs to launch when ``num_sms`` is 0 (afdep/deepep.py:303-306)."""
        if self.num_sms:
            return self.num_sms
        return max(MIN_COMM_SMS, round(device_sms * DEFAULT_COMM_SM_FRACTION))
