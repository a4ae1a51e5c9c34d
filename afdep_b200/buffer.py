"""Public role API: ``Buffer`` with its four calls, receipts, and the low-level facade.

Attention ranks call ``source_dispatch`` then ``source_collect``; FFN ranks call
``worker_receive``, run their experts, then ``worker_reply``.  The contract (tensor shapes,
error messages, one pending exchange per Buffer, collective construction and ``close``)
follows the reference's ``afdep/deepep.py`` and ``docs/api.md``; the machinery underneath
does not.  Roles are native here: an attention rank owns no receive arena and an FFN rank
never originates tokens, so there are no dummy expert slots to route around.

Three transports implement the same five operations:

``native``  sm_100a kernels over the symmetric NVLink heap (`parallel/native_transport.py`)
``gloo``    pure torch over a CPU Gloo group — the oracle and the CPU baseline
``nccl``    ``torch.distributed`` all-to-all over NCCL — the baseline the kernels must beat

This module imports neither torch nor the native library at import time.
"""

from __future__ import annotations

import os
from dataclasses import asdict, dataclass, field
from typing import TYPE_CHECKING, Any, Literal

from .config import (
    FP8_GROUP_SIZE,
    HIDDEN_ALIGNMENT,
    INT32_MAX,
    MAX_EXPERTS_PER_RANK,
    MAX_LOGICAL_EXPERTS,
    MAX_RANKS,
    MAX_TOP_K,
    Config,
)

if TYPE_CHECKING:  # pragma: no cover
    import torch
    import torch.distributed as dist


class AfdepError(RuntimeError):
    """Base class of errors reported by the device side of a Buffer."""


class AfdepTimeoutError(AfdepError):
    """A bounded device wait ran out; the Buffer can only be closed afterwards."""


class AfdepRouteError(AfdepError):
    """A token carried an expert id outside [-1, num_experts) or a repeated expert."""


@dataclass(frozen=True)
class DispatchHandle:
    """Receipt of one dispatch.  Hand it back unchanged with the matching reply."""

    num_experts: int
    num_max_tokens_per_rank: int
    num_sms: int
    recv_shape: tuple[int, int]
    num_tokens: int = 0
    recv_src_metadata: Any = field(default=None, repr=False)   # int32 [rows, 2]: source, token
    _owner: object = field(default=None, repr=False)


@dataclass(frozen=True)
class ReceiveResult:
    """Expert-major rows of one exchange; rows outside the segments are unspecified."""

    recv_x: Any
    recv_scale: Any
    recv_topk_weights: Any
    recv_count_psum: Any
    recv_counts_host: list[int]
    handle: DispatchHandle

    @property
    def receipt(self) -> DispatchHandle:
        return self.handle


def _make_transport(kind: str, **kwargs):
    if kind == "native":
        from .parallel.native_transport import NativeTransport

        return NativeTransport(**kwargs)
    if kind == "gloo":
        from .parallel.gloo_transport import GlooTransport

        return GlooTransport(**kwargs)
    if kind == "nccl":
        from .parallel.nccl_baseline import NcclBaselineTransport

        return NcclBaselineTransport(**kwargs)
    raise ValueError("backend must be 'native', 'gloo' or 'nccl'")


class ElasticBuffer:
    """Union-rank view of the transport, kept for callers of the reference's low-level class.

    ``dispatch`` and ``combine`` are collective over all ranks of the group: attention ranks
    pass their tokens, FFN ranks pass zero rows (afdep/deepep.py:391-512).  ``num_experts``
    counts logical experts, ``world_size * experts_per_rank``, as the reference's class does.
    ``ffn_ranks`` is required: this transport has no symmetric every-rank-is-both mode;
    ``role_aware=False`` only restores the reference's larger receive bound.
    """

    def __init__(
        self,
        *,
        group: "dist.ProcessGroup",
        capacity_tokens_per_rank: int,
        hidden_size: int,
        num_experts: int,
        top_k: int,
        allow_hybrid_mode: bool,
        rdma_traffic_class: int,
        cpu_timeout_s: int,
        gpu_timeout_s: int,
        use_fp8_dispatch: bool = False,
        num_sms: int = 0,
        num_qps: int = 0,
        role_aware: bool = False,
        ffn_ranks: int | None = None,
        expert_alignment: int = 128,
        backend: str = "native",
        scale_format: str = "fp32",
        _control=None,
        _transport_options: dict | None = None,
    ) -> None:
        from .parallel.control import make_control

        self._control = _control if _control is not None else make_control(group)
        self._group = group
        self.rank, self.world_size = self._control.rank, self._control.size
        self.capacity_tokens_per_rank = capacity_tokens_per_rank
        self.num_experts, self.hidden_size, self.top_k = num_experts, hidden_size, top_k
        self.allow_hybrid_mode, self._fp8 = allow_hybrid_mode, use_fp8_dispatch
        self.role_aware, self.ffn_ranks = role_aware, ffn_ranks
        self.backend = backend
        self._owner, self._pending, self._closed = object(), None, False
        self.last_event = None      # EventHandle of the last call made with async_finish=True
        self._transport = None
        settings = {
            "capacity": capacity_tokens_per_rank,
            "hidden": hidden_size,
            "experts": num_experts,
            "top_k": top_k,
            "hybrid": allow_hybrid_mode,
            "traffic_class": rdma_traffic_class,
            "cpu_timeout": cpu_timeout_s,
            "gpu_timeout": gpu_timeout_s,
            "fp8": use_fp8_dispatch,
            "num_sms": num_sms,
            "num_qps": num_qps,
            "role_aware": role_aware,
            "ffn_ranks": ffn_ranks,
            "alignment": expert_alignment,
            "backend": backend,
            "scale_format": scale_format,
        }
        error, probe = None, {}
        try:
            self._preflight(settings)
            probe = self._control.local_probe(backend)
            if num_sms > probe.get("sms", INT32_MAX):
                raise ValueError("num_sms exceeds the selected device SM count")
        except Exception as exc:  # gathered below so that every rank fails together
            error = f"{type(exc).__name__}: {exc}"
        records = self._control.all_gather(
            {"settings": settings, "source": probe.get("source", ""), "error": error, "sms": probe.get("sms", 0)}
        )
        failures = [f"rank {i}: {r['error']}" for i, r in enumerate(records) if r["error"]]
        if failures:
            self._closed = True
            raise RuntimeError("afdep preflight failed: " + "; ".join(failures))
        for key in ("settings", "source"):
            if any(r[key] != records[0][key] for r in records):
                self._closed = True
                raise ValueError(f"Every rank must use the same {key}")
        experts_local = num_experts // self.world_size
        self._experts_local = experts_local
        self._real_experts = experts_local * ffn_ranks
        self._expert_alignment = expert_alignment
        self.device = probe.get("device")
        min_sms = min(r["sms"] for r in records)
        self._config = Config(
            capacity_tokens_per_rank,
            hidden_size,
            self._real_experts,
            top_k,
            ffn_ranks,
            self.world_size - ffn_ranks,
            expert_alignment=expert_alignment,
            payload="fp8" if use_fp8_dispatch else "bf16",
            allow_hybrid_mode=allow_hybrid_mode,
            num_sms=num_sms,
            num_qps=num_qps,
            rdma_traffic_class=rdma_traffic_class,
            cpu_timeout_s=cpu_timeout_s,
            gpu_timeout_s=gpu_timeout_s,
            role_aware=role_aware,
            scale_format=scale_format,
        )
        self._resolved_num_sms = self._config.resolved_num_sms(min_sms) if min_sms else num_sms
        self._transport = _make_transport(
            backend,
            control=self._control,
            group=group,
            config=self._config,
            num_sms=self._resolved_num_sms,
            options=_transport_options or {},
        )
        self.topk_idx_dtype = self._transport.topk_idx_dtype
        self.num_buffer_bytes = self._transport.num_buffer_bytes
        # One NVLink domain holding every rank; there is no scale-out dimension here.
        self.physical_domain = (1, self.world_size)
        self.logical_domain = (1, self.world_size)
        self.num_scaleout_ranks, self.num_scaleup_ranks = self.logical_domain

    # ---- construction helpers --------------------------------------------------------
    def _preflight(self, s: dict) -> None:
        if self.world_size < 2 or not 0 <= self.rank < self.world_size:
            raise ValueError("afdep requires a valid group with at least two ranks")
        for key in ("capacity", "hidden", "experts", "top_k", "cpu_timeout", "gpu_timeout", "alignment"):
            if type(s[key]) is not int or not 0 < s[key] < INT32_MAX:
                raise ValueError(f"{key} must be a positive int32 integer")
        for key in ("num_sms", "num_qps"):
            if type(s[key]) is not int or not 0 <= s[key] < INT32_MAX:
                raise ValueError(f"{key} must be a nonnegative int32 integer")
        if type(s["hybrid"]) is not bool or type(s["fp8"]) is not bool or type(s["role_aware"]) is not bool:
            raise ValueError("hybrid, FP8 and role_aware settings must be booleans")
        if s["scale_format"] not in ("fp32", "ue8m0x4") or (s["scale_format"] != "fp32" and not s["fp8"]):
            raise ValueError("scale_format must be 'fp32', or 'ue8m0x4' with FP8 dispatch")
        ffn = s["ffn_ranks"]
        if ffn is not None and (type(ffn) is not int or not 0 < ffn < self.world_size):
            raise ValueError("ffn_ranks must leave positive FFN and source ranks")
        if s["role_aware"] and ffn is None:
            raise ValueError("role_aware requires explicit ffn_ranks")
        if ffn is None:
            raise ValueError("this transport has native roles and requires explicit ffn_ranks")
        if type(s["traffic_class"]) is not int or not 0 <= s["traffic_class"] <= 255:
            raise ValueError("rdma_traffic_class must be an integer in [0,255]")
        if s["hidden"] % HIDDEN_ALIGNMENT or s["top_k"] > min(MAX_TOP_K, s["experts"]):
            raise ValueError("hidden must divide by 256; top_k must be <=32 and <=experts")
        if s["experts"] % self.world_size:
            raise ValueError("num_experts must divide evenly over the group")
        if s["top_k"] > ffn * (s["experts"] // self.world_size):
            raise ValueError("top_k exceeds the real FFN expert count")
        if (
            self.world_size > MAX_RANKS
            or s["experts"] > MAX_LOGICAL_EXPERTS
            or s["experts"] // self.world_size > MAX_EXPERTS_PER_RANK
            or self.world_size * s["capacity"] * s["top_k"] > INT32_MAX
        ):
            raise ValueError("dimensions exceed the supported workspace/index bounds")
        self._control.check_backend(s["backend"])

    @property
    def comm_stream(self):
        """Stream the exchange kernels run on (the caller's current stream by default)."""
        return self._transport.comm_stream

    @property
    def is_ffn(self) -> bool:
        return self.rank < self.ffn_ranks

    def _check_live(self) -> None:
        if self._closed:
            raise RuntimeError("afdep buffer is closed")
        self._transport.check_device()

    def _num_sms(self) -> int:
        return self._resolved_num_sms

    def _raise_device_status(self) -> None:
        """Surface what a kernel reported since the last call (never blocks)."""
        self._transport.raise_status()

    # ---- exchange --------------------------------------------------------------------
    def dispatch(self, x, x_scale, topk_ids, topk_weights, *, bucket: int, expert_alignment: int, do_cpu_sync: bool,
                 async_finish: bool = False) -> ReceiveResult:
        self._check_live()
        if self._pending is not None:
            raise RuntimeError("Complete the previous exchange before dispatch")
        if type(bucket) is not int or not 0 < bucket <= self.capacity_tokens_per_rank:
            raise ValueError("bucket must be positive and within capacity")
        if type(expert_alignment) is not int or expert_alignment < 1:
            raise ValueError("expert_alignment must be a positive integer")
        if expert_alignment != self._expert_alignment:
            raise ValueError("expert_alignment differs from the one the buffer was built with")
        if type(do_cpu_sync) is not bool:
            raise ValueError("do_cpu_sync must be a boolean")
        if do_cpu_sync and self._transport.is_capturing():
            raise RuntimeError("Host receive counts are unavailable during CUDA capture")
        if x.shape[0] > bucket:
            raise ValueError("source input exceeds its bucket")
        if self.is_ffn and x.shape[0] != 0:
            raise ValueError("role-aware FFN ranks cannot originate tokens")
        if async_finish and self.backend != "native":
            raise ValueError("async_finish needs the native transport")
        self._raise_device_status()
        num_sms = self._num_sms()
        if self.is_ffn:
            out = self._transport.worker_receive(bucket=bucket, read_host_counts=do_cpu_sync)
            recv_x, recv_scale, recv_w, psum, counts, src_meta = out
            n_tokens = 0
        else:
            if async_finish:
                self.last_event = self._transport.source_dispatch(x, x_scale, topk_ids, topk_weights, bucket=bucket, async_finish=True)
            else:
                self._transport.source_dispatch(x, x_scale, topk_ids, topk_weights, bucket=bucket)
            recv_x, recv_scale, recv_w, psum, src_meta = self._transport.empty_receive()
            counts = [0] * self._experts_local if do_cpu_sync else []
            n_tokens = int(x.shape[0])
        handle = DispatchHandle(
            self.num_experts, bucket, num_sms, tuple(recv_x.shape), n_tokens, src_meta, self._owner
        )
        self._pending = handle
        return ReceiveResult(recv_x, recv_scale, recv_w, psum, list(counts), handle)

    def combine(self, expert_output, handle: DispatchHandle, *, async_finish: bool = False):
        self._check_live()
        if handle is None or handle._owner is not self._owner or handle is not self._pending:
            raise ValueError("Handle does not belong to this pending exchange")
        if tuple(expert_output.shape) != handle.recv_shape:
            raise ValueError("Expert output must match its dispatch receive shape")
        if self.is_ffn:
            if async_finish:
                self.last_event = self._transport.worker_reply(expert_output, async_finish=True)
            else:
                self._transport.worker_reply(expert_output)
            combined = self._transport.empty_output()
        else:
            combined = self._transport.source_collect(handle.num_tokens)
        self._pending = None
        return combined

    def close(self) -> None:
        """Collective, outside capture, after every rank's pairs have finished."""
        if self._closed:
            return
        self._check_live()
        if self._transport.is_capturing():
            raise RuntimeError("Close afdep buffers outside CUDA graph capture")
        if any(self._control.all_gather(self._pending is not None)):
            raise RuntimeError("Finish every rank's pending exchange before collective close")
        self._transport.close()
        self._closed = True

    destroy = close


class Buffer:
    """AFD roles, FFN ranks first, one exchange in flight.

    Route only real experts ``[0, num_experts)``, ``-1`` for unused choices, no expert twice
    in a token.  Pass BF16 activations, or e4m3 activations with fp32 per-128 scales
    (``x_scale`` may be a strided view).  Expert rows must be multiplied by
    ``recv_topk_weights`` exactly once before ``worker_reply``.

    Every rank uses the same ``Config``, ``bucket`` and ``read_host_counts`` per exchange.
    Construction and ``close`` are collective and must happen outside CUDA graph capture;
    complete dispatch/reply pairs with ``read_host_counts=False`` may be captured.  The
    caller owns ``group`` (a CPU Gloo group for ``backend="native"`` and ``"gloo"``).

    An illegal route does not trap the GPU: the token publishes nothing, its output row is
    zero, and the next call on this Buffer raises ``AfdepRouteError``.
    """

    def __init__(self, *, group: "dist.ProcessGroup", config: Config, backend: str | None = None, _control=None, **options) -> None:
        from .parallel.control import make_control

        self.config = config
        control = _control if _control is not None else make_control(group)
        configs = control.all_gather(asdict(config))
        if any(value != configs[0] for value in configs):
            raise ValueError("Every AFD rank must use the same Config")
        if control.size != config.world_size:
            raise ValueError("group size does not match the configured AFD topology")
        self.rank = control.rank
        self.role: Literal["ffn", "attention"] = "ffn" if self.rank < config.ffn_ranks else "attention"
        self.role_rank = self.rank if self.role == "ffn" else self.rank - config.ffn_ranks
        backend = backend or os.environ.get("AFDEP_BACKEND", "native")
        self.transport = ElasticBuffer(
            group=group,
            capacity_tokens_per_rank=config.capacity_tokens_per_rank,
            hidden_size=config.hidden_size,
            num_experts=config.logical_experts,
            top_k=config.top_k,
            allow_hybrid_mode=config.allow_hybrid_mode,
            rdma_traffic_class=config.rdma_traffic_class,
            cpu_timeout_s=config.cpu_timeout_s,
            gpu_timeout_s=config.gpu_timeout_s,
            use_fp8_dispatch=config.payload == "fp8",
            scale_format=config.scale_format,
            num_sms=config.num_sms,
            num_qps=config.num_qps,
            role_aware=config.role_aware,
            ffn_ranks=config.ffn_ranks,
            expert_alignment=config.expert_alignment,
            backend=backend,
            _control=control,
            _transport_options=options,
        )
        self.backend = backend
        self.physical_domain = self.transport.physical_domain
        self.logical_domain = self.transport.logical_domain
        self.num_buffer_bytes = self.transport.num_buffer_bytes
        self.topk_idx_dtype = self.transport.topk_idx_dtype
        self.device = self.transport.device
        self._t = self.transport._transport
        self._payload_dtype = self._t.payload_dtype

    # ---- checks ----------------------------------------------------------------------
    def _check_role(self, role: str) -> None:
        self.transport._check_live()
        if self.role != role:
            raise RuntimeError(f"This operation requires the {role} role")

    def _tensor(self, tensor, dtype, shape: tuple[int, ...], *, contiguous: bool = True) -> None:
        if (
            not self._t.on_device(tensor)
            or tensor.dtype != dtype
            or tuple(tensor.shape) != shape
            or (contiguous and not tensor.is_contiguous())
        ):
            raise ValueError("Payload tensor dtype, shape, device or contiguity mismatch")

    @property
    def comm_stream(self):
        return self.transport.comm_stream

    # ---- the four role calls ---------------------------------------------------------
    def source_dispatch(self, x, ids, weights, x_scale=None, *, bucket: int, read_host_counts: bool = False, async_finish: bool = False):
        """Attention: publish activations and expert ids.  No casts, no copies.

        ``async_finish=True`` (native transport built with ``use_comm_stream=True``): the current
        stream does not wait for the dispatch kernel; the call returns an ``EventHandle`` and the
        inputs must not be changed until ``handle.current_stream_wait()`` (or ``synchronize()``)."""
        self._check_role("attention")
        c = self.config
        if x.ndim != 2:
            raise ValueError("source input must have shape [tokens,hidden]")
        n = x.shape[0]
        self._tensor(x, self._payload_dtype, (n, c.hidden_size))
        self._tensor(ids, self.topk_idx_dtype, (n, c.top_k))
        self._tensor(weights, self._t.float32, (n, c.top_k))
        if (x_scale is not None) != (c.payload == "fp8"):
            raise ValueError("FP8 dispatch requires FP32 block128 scales")
        if x_scale is not None:
            if c.scale_packed:      # exponent bytes, four to an int32 word
                self._tensor(x_scale, self._t.scale_dtype, (n, c.scale_groups), contiguous=False)
            else:
                self._tensor(x_scale, self._t.float32, (n, c.hidden_size // FP8_GROUP_SIZE), contiguous=False)
        if not async_finish:
            self.transport.dispatch(x, x_scale, ids, weights, bucket=bucket, expert_alignment=c.expert_alignment, do_cpu_sync=read_host_counts)
            return None
        self.transport.dispatch(x, x_scale, ids, weights, bucket=bucket, expert_alignment=c.expert_alignment, do_cpu_sync=read_host_counts,
                                async_finish=True)
        return self.transport.last_event

    def worker_receive(self, *, bucket: int, read_host_counts: bool = False) -> ReceiveResult:
        """FFN: expert-major rows, weights, device prefix sums and the receipt."""
        self._check_role("ffn")
        e = self._t.empty_source()
        return self.transport.dispatch(
            e[0], e[1], e[2], e[3], bucket=bucket, expert_alignment=self.config.expert_alignment, do_cpu_sync=read_host_counts
        )

    def source_collect(self):
        """Attention: BF16 [T, H], each token's rows summed, in original token order."""
        self._check_role("attention")
        handle = self.transport._pending
        if handle is None:
            raise RuntimeError("source_collect requires a matching dispatch")
        return self.transport.combine(self._t.empty_output(), handle)

    def worker_reply(self, rows, receipt: DispatchHandle, *, async_finish: bool = False):
        """FFN: BF16 rows of the receive shape, weighted exactly once.  ``async_finish=True``
        returns an ``EventHandle`` instead of making the current stream wait (see ``source_dispatch``)."""
        self._check_role("ffn")
        self._tensor(rows, self._t.bfloat16, receipt.recv_shape)
        if not async_finish:
            self.transport.combine(rows, receipt)
            return None
        self.transport.combine(rows, receipt, async_finish=True)
        return self.transport.last_event

    def worker_serve_fused(self, weights, *, bucket: int):
        """FFN, native transport: receive, SwiGLU experts and reply of one exchange as one call.

        ``weights`` is an ``afdep_b200.models.moe_layer.ExpertWeights``.  The received rows are
        never copied into an expert-major ``recv_x``: the gate|up GEMM gathers them from the wire
        records as their arrival flags land.  Returns ``(ReceiveResult, rows)`` where ``recv_x`` and
        ``recv_scale`` are ``None`` and ``rows`` are the BF16 rows that went into the reply.  An
        extension: the reference leaves the experts to its caller (README.md:54-56)."""
        self._check_role("ffn")
        t = self.transport
        if t._pending is not None:
            raise RuntimeError("Complete the previous exchange before dispatch")
        if type(bucket) is not int or not 0 < bucket <= self.config.capacity_tokens_per_rank:
            raise ValueError("bucket must be positive and within capacity")
        if not hasattr(self._t, "worker_mlp_fused"):
            raise RuntimeError("the fused expert path needs the native transport")
        t._raise_device_status()
        psum, recv_w, recv_src, rows = self._t.worker_mlp_fused(weights, bucket=bucket)
        handle = DispatchHandle(t.num_experts, bucket, t._num_sms(), tuple(rows.shape), 0, recv_src, t._owner)
        return ReceiveResult(None, None, recv_w, psum, [], handle), rows

    def check(self) -> None:
        """Raise now if a kernel of this Buffer has reported an error (does not synchronise)."""
        self.transport._raise_device_status()

    def stats(self) -> dict:
        """Registered bytes, kernels launched so far and the last device status."""
        return self._t.stats()

    def close(self) -> None:
        self.transport.close()


# Names the reference keeps for its earlier connector (afdep/deepep.py:724-725).
DeepEPBuffer = Buffer
DeepEPConfig = Config
