"""Every rank of a Buffer inside one process on one GPU.

A loopback world builds ``world_size`` ordinary ``Buffer`` objects whose heaps all live on
the current device and whose peer tables point at each other.  It exists for two reasons:
the single-GPU ("colocated") point of the benchmark, and GPU tests of the full multi-rank
protocol on a machine that offers one GPU.

Kernels of different ranks wait on each other's flags, and launches on one device are not
guaranteed to overlap, so the caller must issue the role calls in dependency order on one
stream: every ``source_dispatch``, then every ``worker_receive``, the experts, every
``worker_reply``, then every ``source_collect``.  In that order each wait is already
satisfied when its kernel starts.  ``exchange`` does exactly this.
"""

from __future__ import annotations

from ..buffer import Buffer
from ..config import Config
from .control import LocalControl


class LoopbackWorld:
    def __init__(self, config: Config, **options) -> None:
        self.config = config
        opts = dict(options)
        opts["loopback"] = True
        self.buffers: list[Buffer] = []
        for rank in range(config.world_size):
            control = LocalControl(rank, config.world_size)
            self.buffers.append(Buffer(group=None, config=config, backend="native", _control=control, **opts))
        transports = [b._t for b in self.buffers]
        for t in transports:
            t.wire_loopback(transports)
        self.ffn = self.buffers[: config.ffn_ranks]
        self.attention = self.buffers[config.ffn_ranks :]

    def exchange(self, batches, expert_fn, *, bucket: int | None = None, read_host_counts: bool = False):
        """One full exchange.  ``batches[a]`` is ``(x, ids, weights, x_scale_or_None)`` for
        attention rank ``a``; ``expert_fn(ffn_role_rank, received) -> rows``.  Returns the
        collected outputs and the FFN ranks' ReceiveResults."""
        bucket = bucket or self.config.capacity_tokens_per_rank
        for buf, (x, ids, w, scale) in zip(self.attention, batches):
            buf.source_dispatch(x, ids, w, scale, bucket=bucket, read_host_counts=read_host_counts)
        received = [buf.worker_receive(bucket=bucket, read_host_counts=read_host_counts) for buf in self.ffn]
        for i, (buf, rec) in enumerate(zip(self.ffn, received)):
            buf.worker_reply(expert_fn(i, rec), rec.receipt)
        outputs = [buf.source_collect() for buf in self.attention]
        return outputs, received

    def close(self) -> None:
        for buf in self.buffers:
            buf.close()
