"""The product transport: sm_100a kernels over a symmetric heap mapped into every peer.

Construction is collective: every rank allocates its heap (CUDA virtual memory exported as a
file descriptor, or a cudaIpc handle when that is unavailable), hands it to every peer over
the control plane, maps the peers' heaps, and meets in a device-side barrier.  After that no
call on the hot path touches the host side of another rank: the four role calls each launch
one kernel (two for ``read_host_counts=True``) on the caller's current stream.
"""

from __future__ import annotations

import os

from ..buffer import AfdepRouteError, AfdepTimeoutError
from ..config import NATIVE_MAX_RANKS, Config


def _env_int(name: str, default: int) -> int:
    value = os.environ.get(name)
    return int(value) if value else default


class EventHandle:
    """What an asynchronous role call hands back: the event that marks the end of the call's
    kernels on the communication stream, plus references that keep the call's tensors alive until
    then.  Counterpart of the reference's EventHandle (csrc/utils/event.hpp:10-42)."""

    def __init__(self, torch_module, event, keep_alive) -> None:
        self._torch, self.event, self._keep_alive = torch_module, event, keep_alive

    def current_stream_wait(self) -> None:
        """Make the current stream wait for the call (a no-op when the call ran on the current stream)."""
        if self.event is not None:
            self._torch.cuda.current_stream().wait_event(self.event)
        self._keep_alive = ()

    def synchronize(self) -> None:
        if self.event is not None:
            self.event.synchronize()
        self._keep_alive = ()

    def query(self) -> bool:
        return True if self.event is None else bool(self.event.query())


class NativeTransport:
    def __init__(self, *, control, group, config: Config, num_sms: int, options: dict) -> None:
        import torch

        from .._native import load_native

        if config.world_size > NATIVE_MAX_RANKS:
            raise ValueError(f"the native transport spans one NVLink domain of at most {NATIVE_MAX_RANKS} ranks")
        self._torch, self._control, self.config = torch, control, config
        self._native = load_native()
        self.device = torch.cuda.current_device()
        bits = int(options.get("topk_idx_bits", os.environ.get("AFDEP_TOPK_IDX_BITS", "64")))
        if bits not in (32, 64):
            raise ValueError("topk_idx_bits must be 32 or 64")
        self.topk_idx_dtype = torch.int64 if bits == 64 else torch.int32
        self.payload_dtype = torch.float8_e4m3fn if config.is_fp8 else torch.bfloat16
        self.float32, self.bfloat16 = torch.float32, torch.bfloat16
        self.scale_dtype = torch.int32 if config.scale_packed else torch.float32      # element type of a row's scales
        self._failed: str | None = None
        self._loopback = bool(options.get("loopback", False))
        # recv_scale comes back column-major with a 4-aligned leading dimension, as the reference
        # always returns it (csrc/elastic/buffer.hpp:1067-1078); "row_major" is the option.
        layout = options.get("recv_scale_layout", "col_major_tma")
        if layout not in ("col_major_tma", "row_major"):
            raise ValueError("recv_scale_layout must be 'col_major_tma' or 'row_major'")
        self._col_major_scale = layout == "col_major_tma"

        timeout_s = float(config.gpu_timeout_s)
        if os.environ.get("AFDEP_TIMEOUT_MS"):
            timeout_s = float(os.environ["AFDEP_TIMEOUT_MS"]) / 1000.0
        if "gpu_timeout_s" in options:
            timeout_s = float(options["gpu_timeout_s"])
        sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        # the collect kernel pulls one token per warp at a time: every SM takes part, as the reference's
        # reduce epilogue does (csrc/kernels/elastic/combine.hpp:248-287), unless the caller caps it
        collect_sms = int(options.get("collect_sms", _env_int("AFDEP_COLLECT_SMS", 0))) or sm_count
        ffn_sms = int(options.get("ffn_sms", _env_int("AFDEP_FFN_SMS", 0))) or sm_count
        bounds = bool(int(os.environ.get("AFDEP_BOUNDS_CHECK", "1")))

        mode = options.get("heap_mode") or os.environ.get("AFDEP_HEAP_MODE")
        if self._loopback:
            mode = "plain"
        elif mode is None:
            mode = "vmm" if self._native.vmm_supported(self.device) else "ipc"
            modes = control.all_gather(mode)
            if any(m != "vmm" for m in modes):
                mode = "ipc"
        self.heap_mode = mode
        self._nb = self._native.NativeBuffer(
            rank=control.rank,
            ffn=config.ffn_ranks,
            attn=config.attention_ranks,
            hidden=config.hidden_size,
            top_k=config.top_k,
            num_experts=config.num_experts,
            capacity=config.capacity_tokens_per_rank,
            fp8=config.is_fp8,
            alignment=config.expert_alignment,
            num_sms=num_sms,
            collect_sms=collect_sms,
            ffn_sms=ffn_sms,
            gpu_timeout_s=timeout_s,
            aux_bytes=int(options.get("aux_bytes", 0)),
            heap_mode=mode,
            bounds_check=bounds,
            p2p_inflight=int(options.get("p2p_inflight", 4)),
            scale_packs=config.scale_groups if config.scale_packed else 0,
        )
        self.num_buffer_bytes = int(self._nb.heap_bytes())
        self.num_sms = num_sms
        self.is_ffn = control.rank < config.ffn_ranks
        self._empty = None
        # Optional running total of rows received per local expert (FFN ranks), accumulated on
        # the device by the receive kernels; read it with ``stats()`` or as ``expert_stats``.
        self.expert_stats = self._nb.enable_expert_stats() if options.get("expert_stats") and self.is_ffn else None
        # Optional dedicated high-priority stream for the exchange kernels, ordered against the
        # caller's current stream with events on both sides of every call (what the reference
        # always does, csrc/elastic/buffer.hpp:476-534).  Off by default: staying on the current
        # stream saves two cross-stream hops per call, which matters at decode latencies.
        want_stream = options.get("use_comm_stream", os.environ.get("AFDEP_COMM_STREAM", "0") not in ("0", ""))
        self._comm_stream = torch.cuda.Stream(device=self.device, priority=-1) if want_stream else None
        self._nvtx = os.environ.get("AFDEP_NVTX", "0") not in ("0", "")
        if not self._loopback:
            self._connect_peers()
            torch.cuda.synchronize(self.device)
            control.barrier()
            self._nb.barrier()
            torch.cuda.synchronize(self.device)
            self.raise_status()

    # ---- bring-up ---------------------------------------------------------------------
    def _connect_peers(self) -> None:
        control, nb = self._control, self._nb
        sizes = control.all_gather(int(nb.mapped_bytes()))
        if self.heap_mode == "vmm":
            from .fd_exchange import exchange_fds

            my_fd = nb.export_fd()
            fds = exchange_fds(control, my_fd)
            try:
                for peer, fd in enumerate(fds):
                    if peer != control.rank:
                        nb.import_peer_fd(peer, fd, sizes[peer])
            finally:
                for fd in fds:
                    if fd >= 0:
                        os.close(fd)
        elif self.heap_mode == "ipc":
            handles = control.all_gather(bytes(nb.export_ipc()))
            for peer, handle in enumerate(handles):
                if peer != control.rank:
                    nb.import_peer_ipc(peer, handle)
        else:
            raise ValueError("a multi-process buffer needs heap_mode 'vmm' or 'ipc'")

    def wire_loopback(self, peers: list["NativeTransport"]) -> None:
        """Loopback world: all heaps live in this process; exchange raw pointers."""
        for peer, other in enumerate(peers):
            if other is not self:
                self._nb.set_peer_ptr(peer, other._nb.local_ptr())

    # ---- small queries ----------------------------------------------------------------
    @property
    def comm_stream(self):
        return self._comm_stream if self._comm_stream is not None else self._torch.cuda.current_stream(self.device)

    def _ranged(self, name: str, fn):
        """NVTX range around a role call when AFDEP_NVTX=1 (for timelines; off by default)."""
        if not self._nvtx:
            return fn()
        self._torch.cuda.nvtx.range_push(f"afdep.{name}")
        try:
            return fn()
        finally:
            self._torch.cuda.nvtx.range_pop()

    def _on_comm_stream(self, fn, *tensors, async_finish: bool = False):
        """Run ``fn`` on the communication stream, after everything queued on the current stream,
        and make the current stream wait for it.  Tensors used by ``fn`` are recorded on the
        communication stream so the caching allocator does not recycle them early.  With
        ``async_finish`` the current stream does *not* wait: the caller gets ``(result, EventHandle)``
        and joins later with ``handle.current_stream_wait()``."""
        if self._comm_stream is None:
            out = fn()
            return (out, EventHandle(self._torch, None, ())) if async_finish else out
        torch = self._torch
        current = torch.cuda.current_stream(self.device)
        self._comm_stream.wait_stream(current)
        with torch.cuda.stream(self._comm_stream):
            out = fn()
        for t in tensors:
            if t is not None and t.numel():
                t.record_stream(self._comm_stream)
        if async_finish:
            done = torch.cuda.Event()
            done.record(self._comm_stream)
            return out, EventHandle(torch, done, tuple(t for t in tensors if t is not None))
        current.wait_stream(self._comm_stream)
        # results were allocated while the communication stream was current but are consumed on
        # the caller's stream: tell the allocator, or a freed block could be reused too early
        stack = [out]
        while stack:
            item = stack.pop()
            if isinstance(item, (tuple, list)):
                stack.extend(item)
            elif isinstance(item, torch.Tensor) and item.is_cuda and item.numel():
                item.record_stream(current)
        return out

    def check_device(self) -> None:
        if self._torch.cuda.current_device() != self.device:
            raise RuntimeError("afdep buffer used on a different CUDA device")

    def is_capturing(self) -> bool:
        return self._torch.cuda.is_current_stream_capturing()

    def on_device(self, tensor) -> bool:
        return bool(tensor.is_cuda) and tensor.get_device() == self.device

    def raise_status(self) -> None:
        if self._failed:
            raise AfdepTimeoutError(self._failed)
        if self._nb.status_code() == 0 or self.is_capturing():
            return
        st = self._nb.status()
        if st["fatal"]:
            self._failed = (
                f"device wait abandoned on rank {st['rank']}: {st['text']} (kernel {st['kernel']}, peer {st['peer']}, "
                f"epoch {st['epoch']}, expected {st['expected']}, observed {st['observed']}); close the buffer"
            )
            raise AfdepTimeoutError(self._failed)
        n = self._nb.bad_routes()
        self._nb.clear_status()
        raise AfdepRouteError(
            f"{n} illegal route(s): first at token {st['expected']}, choice {st['detail0']}, expert id {st['observed']}; "
            "the affected tokens were not dispatched and collect as zero rows"
        )

    def stats(self) -> dict:
        return {
            "backend": "native",
            "heap_mode": self.heap_mode,
            "registered_bytes": self.num_buffer_bytes,
            "record_bytes": int(self._nb.record_bytes()),
            "launches": int(self._nb.launches()),
            "num_sms": int(self._nb.resolved_num_sms()),
            "status": dict(self._nb.status()),
            **({"expert_rows_received": self.expert_stats.tolist()} if self.expert_stats is not None else {}),
        }

    # ---- role operations --------------------------------------------------------------
    def _empties(self):
        if self._empty is None:
            torch, c = self._torch, self.config
            dev = torch.device("cuda", self.device)
            self._empty = {
                "x": torch.empty((0, c.hidden_size), dtype=self.payload_dtype, device=dev),
                "scale": torch.empty((0, c.scale_groups), dtype=self.scale_dtype, device=dev) if c.is_fp8 else None,
                "ids": torch.empty((0, c.top_k), dtype=torch.int64, device=dev),
                "w": torch.empty((0, c.top_k), dtype=torch.float32, device=dev),
                "out": torch.empty((0, c.hidden_size), dtype=torch.bfloat16, device=dev),
                "recv_w": torch.empty((0,), dtype=torch.float32, device=dev),
                "psum": torch.zeros((c.experts_per_rank,), dtype=torch.int32, device=dev),
                "src": torch.empty((0, 2), dtype=torch.int32, device=dev),
            }
        return self._empty

    def empty_source(self):
        e = self._empties()
        return e["x"], e["scale"], e["ids"], e["w"]

    def empty_receive(self):
        e = self._empties()
        return e["x"], e["scale"], e["recv_w"], e["psum"], e["src"]

    def empty_output(self):
        return self._empties()["out"]

    def source_dispatch(self, x, x_scale, ids, weights, *, bucket: int, async_finish: bool = False):
        if x_scale is not None and self.config.scale_packed:
            x_scale = x_scale.view(self._torch.float32)      # the kernels move 4-byte elements; the words pass through untouched
        out = self._ranged(
            "source_dispatch",
            lambda: self._on_comm_stream(lambda: self._nb.source_dispatch(x, x_scale, ids, weights), x, x_scale, ids, weights, async_finish=async_finish),
        )
        return out[1] if async_finish else None

    def source_collect(self, num_tokens: int):
        return self._ranged("source_collect", lambda: self._on_comm_stream(lambda: self._nb.source_collect(num_tokens)))

    def worker_receive(self, *, bucket: int, read_host_counts: bool):
        rows = self.config.receive_rows(bucket)
        out = self._ranged(
            "worker_receive",
            lambda: self._on_comm_stream(
                lambda: self._nb.worker_receive(rows, read_host_counts, float(self.config.cpu_timeout_s), self._col_major_scale)
            ),
        )
        if self.config.scale_packed and out[1] is not None:
            out = (out[0], out[1].view(self._torch.int32), *out[2:])
        return out

    def worker_mlp_fused(self, weights, *, bucket: int):
        """Layout pass, gathered gate|up GEMM, down GEMM and reply of one exchange; returns
        ``(psum, recv_weights, recv_src, rows)``."""
        fp8 = self.config.is_fp8
        if fp8 and (weights.mode != "fp8" or weights.w_down_scale is None or getattr(weights, "scale_format", "fp32") != "pow2"):
            raise ValueError("the fused expert path takes FP8 payloads only with FP8 experts whose block scales are powers of two")
        if not fp8 and weights.mode != "bf16":
            raise ValueError("the fused expert path takes BF16 payloads only with BF16 experts")
        rows = self.config.receive_rows(bucket)
        tensors = (weights.w_gate_up, weights.w_gate_up_scale, weights.w_down, weights.w_down_scale)
        return self._ranged(
            "worker_mlp_fused",
            lambda: self._on_comm_stream(lambda: self._nb.worker_mlp_fused(tensors[0], tensors[1], tensors[2], tensors[3], rows), *tensors),
        )

    def worker_reply(self, rows, *, async_finish: bool = False):
        out = self._ranged("worker_reply", lambda: self._on_comm_stream(lambda: self._nb.worker_reply(rows), rows, async_finish=async_finish))
        return out[1] if async_finish else None

    def close(self) -> None:
        torch = self._torch
        torch.cuda.synchronize(self.device)
        if not self._loopback:
            self._control.barrier()
            if not self._failed and self._nb.status_code() in (0, 16):
                self._nb.barrier()
                torch.cuda.synchronize(self.device)
            self._control.barrier()
        self._nb.destroy()
