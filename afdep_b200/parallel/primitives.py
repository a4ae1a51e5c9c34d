"""Secondary primitives on a native Buffer's symmetric heap: all-gather, neighbour send/recv
with credits, and remote row fetch.  NVLink only.

They live in the heap's auxiliary region, whose size is chosen when the Buffer is built
(``Buffer(..., aux_bytes=..., p2p_inflight=4)``).  The three primitives share that data area,
one at a time (separate phases with ``barrier()``): an all-gather uses two sets of one slot per
rank, send/recv a ring of ``p2p_inflight`` message slots per source rank, the row fetch this
rank's shard of the table.  The
reference inherits comparable calls from its vendored transport (pipeline send/recv, an
in-session all-gather and an embedding-row fetch, csrc/elastic/buffer.hpp:201-474) without
exposing them in its role API; here they are a thin, explicit layer next to the role API.

Every wait is bounded like the role calls': a peer that never shows up surfaces as
``AfdepTimeoutError`` at the next ``Buffer.check()``.
"""

from __future__ import annotations

import torch


class HeapPrimitives:
    def __init__(self, buffer) -> None:
        if buffer.backend != "native":
            raise ValueError("heap primitives need the native transport")
        self._buffer = buffer
        self._nb = buffer._t._nb
        self.world_size = buffer.config.world_size
        self.rank = buffer.rank
        self._side = None
        if self._nb.aux_slot_bytes() <= 0:
            raise ValueError("build the Buffer with aux_bytes > 0 to use heap primitives")

    @property
    def slot_bytes(self) -> int:
        """Largest tensor a rank can contribute to an all-gather."""
        return int(self._nb.aux_slot_bytes())

    @property
    def message_bytes(self) -> int:
        """Largest send/recv message."""
        return int(self._nb.p2p_slot_bytes())

    @property
    def inflight(self) -> int:
        """Messages a sender can have on their way to one peer before it waits for that peer."""
        return int(self._nb.p2p_inflight())

    # ---- all-gather ---------------------------------------------------------------------
    def all_gather_start(self, tensor: torch.Tensor, *, engine: str = "sm"):
        """Push ``tensor`` into every peer's slot for this rank.  Returns a handle whose
        ``wait()`` yields the gathered data ``[world_size, *tensor.shape]`` as a tensor of its own
        (copied out of the heap on the current stream, so gathers may follow one another without
        a barrier: the slots alternate between two sets and a set is reused only after every
        rank has copied its previous contents out).

        ``engine="sm"`` copies with a kernel (graph-capturable).  ``engine="copy"`` uses one
        copy-engine transfer per peer and a batched stream memory operation for the flags, so
        no SM is occupied while compute kernels run; it is eager-only.  All ranks may choose
        independently: the flags and the bounded wait are the same."""
        if engine == "sm":
            self._nb.allgather_push(tensor)
        elif engine == "copy":
            self._nb.allgather_push_copy(tensor)
        else:
            raise ValueError("engine must be 'sm' or 'copy'")
        return _GatherHandle(self, tensor.shape, tensor.dtype, tensor.numel() * tensor.element_size())

    def all_gather(self, tensor: torch.Tensor, *, engine: str = "sm") -> torch.Tensor:
        return self.all_gather_start(tensor, engine=engine).wait()

    # ---- neighbour send / recv -------------------------------------------------------------
    def send(self, tensor: torch.Tensor, dst: int) -> None:
        """One message to ``dst``.  Up to ``inflight`` messages may be on their way; the kernel of
        message ``n`` waits (bounded, on the device) until ``dst`` has consumed message ``n - inflight``.
        Sends of one Buffer must be stream-ordered among themselves, receives likewise (they number
        their messages on the device); a send may run beside a receive on another stream."""
        self._nb.p2p_send(tensor, int(dst))

    def recv(self, out: torch.Tensor, src: int) -> torch.Tensor:
        """Next message from ``src`` into ``out``; returns the credit to the sender."""
        self._nb.p2p_recv(out, int(src))
        return out

    # ---- remote row fetch ---------------------------------------------------------------------
    def table_shard(self, rows_per_rank: int, row_elems: int, dtype: torch.dtype) -> torch.Tensor:
        """This rank's shard ``[rows_per_rank, row_elems]`` of a table spread over all ranks,
        as a view of the auxiliary data area.  Fill it, then ``Buffer``-barrier before fetching."""
        n = rows_per_rank * row_elems * torch.empty((), dtype=dtype).element_size()
        return self._nb.aux_view()[:n].view(dtype).view(rows_per_rank, row_elems)

    def fetch_rows(self, idx: torch.Tensor, rows_per_rank: int, row_elems: int, dtype: torch.dtype) -> torch.Tensor:
        """Rows ``idx`` (global row numbers, owner = idx // rows_per_rank) gathered over NVLink."""
        row_bytes = row_elems * torch.empty((), dtype=dtype).element_size()
        raw = self._nb.fetch_rows(idx, int(rows_per_rank), int(row_bytes))
        return raw.view(dtype).view(idx.numel(), row_elems)

    def fetch_rows_start(self, idx: torch.Tensor, rows_per_rank: int, row_elems: int, dtype: torch.dtype) -> "_FetchHandle":
        """Issue the same fetch on a side stream and return at once; ``handle.wait()`` makes the
        current stream wait for it and hands over the rows.  Work queued on the current stream
        between the two calls overlaps the transfer (the reference splits its fetch into an
        issue and a wait kernel for the same purpose, impls/engram_fetch.cuh:11-97)."""
        if self._side is None:
            self._side = torch.cuda.Stream(device=idx.device)
        current = torch.cuda.current_stream(idx.device)
        self._side.wait_stream(current)
        with torch.cuda.stream(self._side):
            rows = self.fetch_rows(idx, rows_per_rank, row_elems, dtype)
            done = torch.cuda.Event()
            done.record(self._side)
        idx.record_stream(self._side)
        return _FetchHandle(rows, done)

    def barrier(self) -> None:
        """Device-side barrier over all ranks on the current stream."""
        self._nb.barrier()


class _GatherHandle:
    def __init__(self, owner: HeapPrimitives, shape, dtype, nbytes: int) -> None:
        self._owner, self._shape, self._dtype, self._nbytes = owner, tuple(shape), dtype, nbytes

    def wait(self) -> torch.Tensor:
        o = self._owner
        raw = o._nb.allgather_wait(int(self._nbytes))          # uint8 [world, nbytes], a copy
        return raw.view(self._dtype).view(o.world_size, *self._shape)


class _FetchHandle:
    def __init__(self, rows: torch.Tensor, done) -> None:
        self._rows, self._done = rows, done

    def wait(self) -> torch.Tensor:
        current = torch.cuda.current_stream(self._rows.device)
        current.wait_event(self._done)
        self._rows.record_stream(current)
        return self._rows
