"""The exchange in pure torch over a CPU Gloo group: oracle and CPU baseline.

Same five operations as the CUDA transport, same placement rules
(`afdep_b200.utils.oracle`), point-to-point ``send``/``recv`` between every
(attention, FFN) pair.  Used by the multi-process CPU tests of the host logic and as the
timed CPU baseline; it is deliberately simple rather than fast.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..config import Config
from ..utils import oracle
from ..utils.scales import scale_dtype


class GlooTransport:
    def __init__(self, *, control, group, config: Config, num_sms: int, options: dict) -> None:
        self._control, self._group, self.config = control, group, config
        self.rank = control.rank
        self.is_ffn = self.rank < config.ffn_ranks
        self.role_rank = self.rank if self.is_ffn else self.rank - config.ffn_ranks
        self.device = None
        self.topk_idx_dtype = torch.int64
        self.payload_dtype = torch.float8_e4m3fn if config.is_fp8 else torch.bfloat16
        self.float32, self.bfloat16 = torch.float32, torch.bfloat16
        self.scale_dtype = torch.int32 if config.scale_packed else torch.float32      # element type of a row's scales
        self.num_buffer_bytes = 0
        self._launches = 0
        self._slots = None        # attention: per FFN rank, token index of every record
        self._records = None      # FFN: per source, (token ids [n], rows [n, K] or -1)

    # ---- queries ----------------------------------------------------------------------
    comm_stream = None

    def check_device(self) -> None:
        return None

    def is_capturing(self) -> bool:
        return False

    def on_device(self, tensor) -> bool:
        return not tensor.is_cuda

    def raise_status(self) -> None:
        return None

    def stats(self) -> dict:
        return {"backend": "gloo", "registered_bytes": 0, "launches": self._launches}

    def empty_source(self):
        c = self.config
        return (
            torch.empty((0, c.hidden_size), dtype=self.payload_dtype),
            torch.empty((0, c.scale_groups), dtype=scale_dtype(c)) if c.is_fp8 else None,
            torch.empty((0, c.top_k), dtype=torch.int64),
            torch.empty((0, c.top_k), dtype=torch.float32),
        )

    def empty_receive(self):
        c = self.config
        return (
            torch.empty((0, c.hidden_size), dtype=self.payload_dtype),
            torch.empty((0, c.scale_groups), dtype=scale_dtype(c)) if c.is_fp8 else None,
            torch.empty((0,), dtype=torch.float32),
            torch.zeros((c.experts_per_rank,), dtype=torch.int32),
            torch.empty((0, 2), dtype=torch.int32),
        )

    def empty_output(self):
        return torch.empty((0, self.config.hidden_size), dtype=torch.bfloat16)

    # ---- wire helpers -----------------------------------------------------------------
    def _send(self, tensor: torch.Tensor, dst: int) -> None:
        t = tensor.contiguous()
        if t.dtype == torch.float8_e4m3fn:
            t = t.view(torch.uint8)
        if t.dtype == torch.bfloat16:
            t = t.view(torch.int16)
        if t.numel():
            dist.send(t, dst=dist.get_global_rank(self._group, dst), group=self._group)

    def _recv(self, shape, dtype, src: int) -> torch.Tensor:
        wire = {torch.float8_e4m3fn: torch.uint8, torch.bfloat16: torch.int16}.get(dtype, dtype)
        t = torch.empty(shape, dtype=wire)
        if t.numel():
            dist.recv(t, src=dist.get_global_rank(self._group, src), group=self._group)
        return t.view(dtype) if wire is not dtype else t

    # ---- role operations --------------------------------------------------------------
    def source_dispatch(self, x, x_scale, ids, weights, *, bucket: int) -> None:
        c = self.config
        el = c.experts_per_rank
        legal = oracle.legal_ids(ids, c.num_experts)
        self._slots = []
        for f in range(c.ffn_ranks):
            local = (legal >= f * el) & (legal < (f + 1) * el)
            tokens = torch.nonzero(local.any(dim=1)).flatten()
            counts = oracle.expert_counts(legal, c.num_experts)[f * el : (f + 1) * el]
            header = torch.cat((torch.tensor([tokens.numel()], dtype=torch.int64), counts))
            self._send(header, f)
            sel = torch.where(local[tokens], legal[tokens], torch.full_like(legal[tokens], -1))
            self._send(x[tokens], f)
            if c.is_fp8:
                self._send(x_scale[tokens].contiguous(), f)
            self._send(sel, f)
            self._send(weights[tokens], f)
            self._send(tokens, f)
            self._slots.append(tokens)
        self._launches += 1

    def worker_receive(self, *, bucket: int, read_host_counts: bool):
        c = self.config
        el, K, f = c.experts_per_rank, c.top_k, self.role_rank
        headers, payloads = [], []
        for a in range(c.attention_ranks):
            src = c.ffn_ranks + a
            header = self._recv((1 + el,), torch.int64, src)
            n = int(header[0])
            x = self._recv((n, c.hidden_size), self.payload_dtype, src)
            scale = self._recv((n, c.scale_groups), scale_dtype(c), src) if c.is_fp8 else None
            ids = self._recv((n, K), torch.int64, src)
            w = self._recv((n, K), torch.float32, src)
            tokens = self._recv((n,), torch.int64, src)
            headers.append(header[1:])
            payloads.append((x, scale, ids, w, tokens))
        layout = oracle.ffn_layout(torch.stack(headers), c.expert_alignment)
        rows = layout.rows_exact if read_host_counts else c.receive_rows(bucket)
        recv_x = torch.zeros((rows, c.hidden_size), dtype=self.payload_dtype)
        recv_scale = torch.zeros((rows, c.scale_groups), dtype=scale_dtype(c)) if c.is_fp8 else None
        recv_w = torch.zeros((rows,), dtype=torch.float32)
        recv_src = torch.full((rows, 2), -1, dtype=torch.int32)
        self._records = []
        for a, (x, scale, ids, w, tokens) in enumerate(payloads):
            rec_rows = torch.full(ids.shape, -1, dtype=torch.int64)
            cursor = layout.row_base[a].clone()
            for r in range(ids.shape[0]):          # records arrive in token order
                for k in range(K):
                    e = int(ids[r, k])
                    if e < 0:
                        continue
                    row = int(cursor[e - f * el])
                    cursor[e - f * el] += 1
                    rec_rows[r, k] = row
                    recv_x[row] = x[r]
                    if recv_scale is not None:
                        recv_scale[row] = scale[r]
                    recv_w[row] = w[r, k]
                    recv_src[row, 0], recv_src[row, 1] = a, int(tokens[r])
            self._records.append(rec_rows)
        self._launches += 1
        counts = layout.aligned_counts if read_host_counts else []
        return recv_x, recv_scale, recv_w, layout.ends.to(torch.int32), counts, recv_src

    def worker_reply(self, rows) -> None:
        c = self.config
        rf = rows.float()
        for a, rec_rows in enumerate(self._records):
            n = rec_rows.shape[0]
            out = torch.zeros((n, c.hidden_size), dtype=torch.float32)
            for k in range(rec_rows.shape[1]):      # fp32, in top-k order
                sel = rec_rows[:, k] >= 0
                out[sel] += rf[rec_rows[sel, k]]
            self._send(out.to(torch.bfloat16), c.ffn_ranks + a)
        self._records = None
        self._launches += 1

    def source_collect(self, num_tokens: int):
        c = self.config
        acc = torch.zeros((num_tokens, c.hidden_size), dtype=torch.float32)
        for f, tokens in enumerate(self._slots):
            part = self._recv((tokens.numel(), c.hidden_size), torch.bfloat16, f)
            acc[tokens] += part.float()
        self._slots = None
        self._launches += 1
        return acc.to(torch.bfloat16)

    def close(self) -> None:
        self._control.barrier()
