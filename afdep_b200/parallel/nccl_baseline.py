"""Baseline transport: the same role calls built from NCCL collectives and torch index ops.

This is what the CUDA transport has to beat, not part of it.  Each direction is one
``all_to_all_single`` of counts followed by one of rows over a NCCL group created next to the
caller's Gloo group; permutation, expansion and reduction are ordinary torch kernels
(``nonzero``, ``argsort``, ``index_select``, ``index_add_``), and split sizes go through the
host, as they must with NCCL.  Placement rules and rounding match
`afdep_b200.utils.oracle`, so outputs are interchangeable with the native transport's.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..config import Config
from ..utils.scales import scale_dtype


class NcclBaselineTransport:
    def __init__(self, *, control, group, config: Config, num_sms: int, options: dict) -> None:
        self._control, self.config = control, config
        self.rank, self.world = control.rank, control.size
        self.is_ffn = self.rank < config.ffn_ranks
        self.role_rank = self.rank if self.is_ffn else self.rank - config.ffn_ranks
        self.device = torch.cuda.current_device()
        self._dev = torch.device("cuda", self.device)
        self.topk_idx_dtype = torch.int64
        self.payload_dtype = torch.float8_e4m3fn if config.is_fp8 else torch.bfloat16
        self.float32, self.bfloat16 = torch.float32, torch.bfloat16
        self.scale_dtype = torch.int32 if config.scale_packed else torch.float32      # element type of a row's scales
        self.num_buffer_bytes = 0
        self._launches = 0
        ranks = control.all_gather(dist.get_rank())
        self._nccl = dist.new_group(ranks=ranks, backend="nccl")
        self._state = None
        warm = torch.zeros(self.world, device=self._dev)
        dist.all_reduce(warm, group=self._nccl)
        torch.cuda.synchronize(self.device)

    comm_stream = None

    def check_device(self) -> None:
        if torch.cuda.current_device() != self.device:
            raise RuntimeError("afdep buffer used on a different CUDA device")

    def is_capturing(self) -> bool:
        return torch.cuda.is_current_stream_capturing()

    def on_device(self, tensor) -> bool:
        return bool(tensor.is_cuda) and tensor.get_device() == self.device

    def raise_status(self) -> None:
        return None

    def stats(self) -> dict:
        return {"backend": "nccl", "registered_bytes": 0, "launches": self._launches}

    def _empty(self, shape, dtype):
        return torch.empty(shape, dtype=dtype, device=self._dev)

    def empty_source(self):
        c = self.config
        return (
            self._empty((0, c.hidden_size), self.payload_dtype),
            self._empty((0, c.scale_groups), scale_dtype(c)) if c.is_fp8 else None,
            self._empty((0, c.top_k), torch.int64),
            self._empty((0, c.top_k), torch.float32),
        )

    def empty_receive(self):
        c = self.config
        return (
            self._empty((0, c.hidden_size), self.payload_dtype),
            self._empty((0, c.scale_groups), scale_dtype(c)) if c.is_fp8 else None,
            self._empty((0,), torch.float32),
            torch.zeros((c.experts_per_rank,), dtype=torch.int32, device=self._dev),
            self._empty((0, 2), torch.int32),
        )

    def empty_output(self):
        return self._empty((0, self.config.hidden_size), torch.bfloat16)

    # ---- the two collectives ---------------------------------------------------------
    def _a2a(self, send: torch.Tensor, send_rows: list[int], recv_rows: list[int]) -> torch.Tensor:
        wire = send.view(torch.uint8) if send.dtype == torch.float8_e4m3fn else send
        out = torch.empty((sum(recv_rows), *wire.shape[1:]), dtype=wire.dtype, device=self._dev)
        dist.all_to_all_single(out, wire.contiguous(), recv_rows, send_rows, group=self._nccl)
        return out.view(send.dtype) if wire is not send else out

    def _dispatch(self, x, x_scale, ids, weights):
        c = self.config
        W, F, el, K = self.world, c.ffn_ranks, c.experts_per_rank, c.top_k
        T = x.shape[0]
        # header per destination: [records, counts of its experts]
        header = torch.zeros((W, 1 + el), dtype=torch.int64, device=self._dev)
        order, send_rows = [], [0] * W
        if T:
            dest = torch.where(ids >= 0, ids // el, torch.full_like(ids, -1))
            for f in range(F):
                hit = dest == f
                tok = torch.nonzero(hit.any(dim=1)).flatten()
                order.append(tok)
                header[f, 0] = tok.numel()
                header[f, 1:] = torch.bincount((ids[hit] - f * el), minlength=el)
            send_rows[:F] = [int(v) for v in header[:F, 0].tolist()]      # host sync
        got = torch.empty_like(header)
        dist.all_to_all_single(got, header, group=self._nccl)
        recv_rows = [int(v) for v in got[:, 0].tolist()]                   # host sync
        tok_all = torch.cat(order) if order else torch.empty(0, dtype=torch.int64, device=self._dev)
        payload = self._a2a(x[tok_all], send_rows, recv_rows)
        scale = self._a2a(x_scale[tok_all].contiguous(), send_rows, recv_rows) if c.is_fp8 else None
        rid = self._a2a(ids[tok_all], send_rows, recv_rows)
        rw = self._a2a(weights[tok_all], send_rows, recv_rows)
        rtok = self._a2a(tok_all, send_rows, recv_rows)
        self._launches += 6
        return got, recv_rows, send_rows, order, payload, scale, rid, rw, rtok

    def source_dispatch(self, x, x_scale, ids, weights, *, bucket: int) -> None:
        out = self._dispatch(x, x_scale, ids, weights)
        self._state = {"send_rows": out[2], "order": out[3], "T": x.shape[0]}

    def worker_receive(self, *, bucket: int, read_host_counts: bool):
        c = self.config
        el, K, f, A = c.experts_per_rank, c.top_k, self.role_rank, c.attention_ranks
        e = self.empty_source()
        got, recv_rows, _, _, payload, scale, rid, rw, rtok = self._dispatch(*e)
        counts = got[c.ffn_ranks :, 1:]                                     # [A, el]
        totals = counts.sum(dim=0)
        aligned = (totals + c.expert_alignment - 1) // c.expert_alignment * c.expert_alignment
        starts = torch.cumsum(aligned, 0) - aligned
        ends = starts + totals
        row_base = starts[None, :] + torch.cumsum(counts, 0) - counts
        aligned_host = [int(v) for v in aligned.tolist()] if read_host_counts else []
        rows = sum(aligned_host) if read_host_counts else c.receive_rows(bucket)
        src_of = torch.repeat_interleave(torch.arange(self.world, device=self._dev), torch.tensor(recv_rows, device=self._dev)) - c.ffn_ranks
        local = (rid >= f * el) & (rid < (f + 1) * el)
        r_idx, k_idx = torch.nonzero(local, as_tuple=True)                   # (record, k) order
        e_loc = rid[r_idx, k_idx] - f * el
        a_idx = src_of[r_idx]
        key = (a_idx * el + e_loc) * (rid.numel() + 1) + r_idx * K + k_idx
        order = torch.argsort(key)
        grp = (a_idx * el + e_loc)[order]
        first = torch.searchsorted(grp, grp)
        pos = torch.arange(order.numel(), device=self._dev) - first
        dst = torch.empty_like(order)
        dst[order] = row_base.flatten()[grp] + pos
        recv_x = self._empty((rows, c.hidden_size), self.payload_dtype)
        recv_w = self._empty((rows,), torch.float32)
        recv_src = torch.full((rows, 2), -1, dtype=torch.int32, device=self._dev)
        if self.payload_dtype == torch.float8_e4m3fn:
            recv_x.view(torch.uint8)[dst] = payload.view(torch.uint8)[r_idx]
        else:
            recv_x[dst] = payload[r_idx]
        recv_scale = None
        if c.is_fp8:
            recv_scale = self._empty((rows, c.scale_groups), scale_dtype(c))
            recv_scale[dst] = scale[r_idx]
        recv_w[dst] = rw[r_idx, k_idx]
        recv_src[dst, 0] = a_idx.to(torch.int32)
        recv_src[dst, 1] = rtok[r_idx].to(torch.int32)
        self._state = {"recv_rows": recv_rows, "r_idx": r_idx, "dst": dst, "n_rec": rid.shape[0]}
        self._launches += 20
        return recv_x, recv_scale, recv_w, ends.to(torch.int32), aligned_host, recv_src

    def worker_reply(self, rows) -> None:
        c, st = self.config, self._state
        reduced = torch.zeros((st["n_rec"], c.hidden_size), dtype=torch.float32, device=self._dev)
        reduced.index_add_(0, st["r_idx"], rows[st["dst"]].float())
        self._a2a(reduced.to(torch.bfloat16), st["recv_rows"], [0] * self.world)
        self._state = None
        self._launches += 4

    def source_collect(self, num_tokens: int):
        c, st = self.config, self._state
        empty = self._empty((0, c.hidden_size), torch.bfloat16)
        back = self._a2a(empty, [0] * self.world, st["send_rows"])
        acc = torch.zeros((num_tokens, c.hidden_size), dtype=torch.float32, device=self._dev)
        offset = 0
        for tok in st["order"]:                       # FFN rank order
            part = back[offset : offset + tok.numel()]
            offset += tok.numel()
            acc.index_add_(0, tok, part.float())
        self._state = None
        self._launches += 4
        return acc.to(torch.bfloat16)

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        self._control.barrier()
        dist.destroy_process_group(self._nccl)
