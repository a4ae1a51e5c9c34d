"""Pure-torch statement of what one exchange must compute.  Runs anywhere, on any device.

Everything the CUDA kernels do is checked against these functions, and the Gloo transport
(`afdep_b200.parallel.gloo_transport`) is built from them.  The reference has no CPU
implementation of its transport (its unit tests mock the native module,
tests/unit/test_deepep.py:2), so this file is also the definition of the semantics:

1. ``cnt[a][e]``: choices of expert ``e`` by source ``a``; ``-1`` choices are skipped; a token
   with an id outside ``[-1, num_experts)`` or a repeated expert is illegal and publishes
   nothing.
2. On FFN rank ``f`` (experts ``[f*E_l, (f+1)*E_l)``): ``start[e]`` is the running sum of the
   totals of the earlier local experts, each rounded up to ``expert_alignment``;
   ``ends[e] = start[e] + total[e]``; inside a segment rows are ordered by
   (source rank, token, k).
3. The caller produces one BF16 row per received row, already multiplied by the routing weight.
4. ``out[a][t]`` is the sum of the token's rows.  The transport reduces in two stages: rows
   that sit on the same FFN rank are added in fp32 (in top-k order) and rounded to BF16 once,
   then the per-rank rows are added in fp32 in rank order and rounded again.  A stage with a
   single addend is an exact copy.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..config import Config, align_up


def legal_ids(ids: torch.Tensor, num_experts: int) -> torch.Tensor:
    """ids with every choice of an illegal token replaced by -1."""
    ids = ids.to(torch.int64)
    bad = (ids < -1) | (ids >= num_experts)
    if ids.shape[1] > 1:
        srt, _ = torch.sort(ids, dim=1)
        dup = ((srt[:, 1:] == srt[:, :-1]) & (srt[:, 1:] >= 0)).any(dim=1)
    else:
        dup = torch.zeros(ids.shape[0], dtype=torch.bool, device=ids.device)
    illegal = bad.any(dim=1) | dup
    return torch.where(illegal[:, None], torch.full_like(ids, -1), ids)


def illegal_tokens(ids: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Boolean mask of tokens the route guard rejects."""
    ids = ids.to(torch.int64)
    bad = ((ids < -1) | (ids >= num_experts)).any(dim=1)
    srt, _ = torch.sort(ids, dim=1)
    dup = ((srt[:, 1:] == srt[:, :-1]) & (srt[:, 1:] >= 0)).any(dim=1) if ids.shape[1] > 1 else torch.zeros_like(bad)
    return bad | dup


def expert_counts(ids: torch.Tensor, num_experts: int) -> torch.Tensor:
    """int64 [num_experts]: how often each expert is chosen (ids already legal)."""
    flat = ids[ids >= 0].to(torch.int64)
    return torch.bincount(flat, minlength=num_experts)[:num_experts]


@dataclass
class FfnLayout:
    totals: torch.Tensor      # [E_l]
    starts: torch.Tensor      # [E_l] aligned segment starts
    ends: torch.Tensor        # [E_l] start + total  (this is recv_count_psum)
    row_base: torch.Tensor    # [A][E_l] first row of (source, expert)
    aligned_counts: list[int]  # what read_host_counts reports
    rows_exact: int           # sum of aligned counts


def ffn_layout(counts: torch.Tensor, alignment: int) -> FfnLayout:
    """counts: int64 [A][E_l] for one FFN rank."""
    counts = counts.to(torch.int64).cpu()
    totals = counts.sum(dim=0)
    aligned = (totals + alignment - 1) // alignment * alignment
    starts = torch.cumsum(aligned, 0) - aligned
    ends = starts + totals
    row_base = starts[None, :] + torch.cumsum(counts, 0) - counts
    return FfnLayout(totals, starts, ends, row_base, [int(v) for v in aligned], int(aligned.sum()))


@dataclass
class SourceBatch:
    """Inputs of one attention rank for one exchange."""

    x: torch.Tensor                    # [T, H] bf16 or e4m3
    ids: torch.Tensor                  # [T, K] int64
    weights: torch.Tensor              # [T, K] fp32
    x_scale: torch.Tensor | None = None   # [T, H/128] fp32 (any strides)


@dataclass
class ExpectedReceive:
    recv_x: torch.Tensor            # [rows, H], padding rows zero
    recv_scale: torch.Tensor | None
    recv_weights: torch.Tensor      # [rows]
    recv_src: torch.Tensor          # [rows, 2] (source, token), -1 in padding
    valid: torch.Tensor             # [rows] bool
    layout: FfnLayout


def expected_receive(config: Config, ffn_rank: int, sources: list[SourceBatch], rows: int | None = None) -> ExpectedReceive:
    """What ``worker_receive`` must return on ``ffn_rank`` (valid rows only are specified)."""
    el = config.experts_per_rank
    lo = ffn_rank * el
    legal = [legal_ids(s.ids, config.num_experts).cpu() for s in sources]
    counts = torch.stack([expert_counts(i, config.num_experts)[lo : lo + el] for i in legal])
    layout = ffn_layout(counts, config.expert_alignment)
    if rows is None:
        rows = layout.rows_exact
    x0 = sources[0].x
    recv_x = torch.zeros((rows, config.hidden_size), dtype=x0.dtype)
    recv_scale = torch.zeros((rows, config.scale_groups), dtype=torch.int32 if config.scale_packed else torch.float32) if config.is_fp8 else None
    recv_w = torch.zeros((rows,), dtype=torch.float32)
    recv_src = torch.full((rows, 2), -1, dtype=torch.int32)
    valid = torch.zeros((rows,), dtype=torch.bool)
    for a, (src, ids) in enumerate(zip(sources, legal)):
        x = src.x.cpu()
        w = src.weights.cpu()
        sc = src.x_scale.cpu() if src.x_scale is not None else None
        t_idx, k_idx = torch.nonzero((ids >= lo) & (ids < lo + el), as_tuple=True)   # (token, k) order
        e_loc = ids[t_idx, k_idx] - lo
        # position among this source's choices of the same expert, in (token, k) order
        order = torch.argsort(e_loc * (ids.numel() + 1) + t_idx * ids.shape[1] + k_idx)
        e_sorted = e_loc[order]
        first = torch.searchsorted(e_sorted, e_sorted)
        pos_sorted = torch.arange(order.numel()) - first
        rows_idx = torch.empty_like(order)
        rows_idx[order] = layout.row_base[a][e_sorted] + pos_sorted
        recv_x[rows_idx] = x[t_idx]
        if recv_scale is not None:
            recv_scale[rows_idx] = sc[t_idx]
        recv_w[rows_idx] = w[t_idx, k_idx]
        recv_src[rows_idx, 0] = a
        recv_src[rows_idx, 1] = t_idx.to(torch.int32)
        valid[rows_idx] = True
    return ExpectedReceive(recv_x, recv_scale, recv_w, recv_src, valid, layout)


def dequantize(x: torch.Tensor, scale: torch.Tensor | None) -> torch.Tensor:
    """fp32 view of a payload: e4m3 rows times their per-128 scales (fp32, or int32 words of
    packed exponent bytes), or bf16 rows."""
    xf = x.float()
    if scale is None:
        return xf
    rows, hidden = xf.shape
    if scale.dtype == torch.int32:        # exponent bytes packed four to a word
        from .scales import unpack_ue8m0x4

        scale = unpack_ue8m0x4(scale, hidden // 128)
    return (xf.view(rows, hidden // 128, 128) * scale.float()[:, :, None]).reshape(rows, hidden)


def synthetic_expert_rows(config: Config, ffn_rank: int, recv_x, recv_scale, recv_weights, ends: torch.Tensor) -> torch.Tensor:
    """The test "expert": expert ``e`` multiplies by ``e + 1``; rows are weighted once.

    Rows outside every segment are zero.  Mirrors the reference's GPU test helper
    (tests/gpu/deepep.py:69-88) so that results stay exactly representable in BF16.
    """
    el, align = config.experts_per_rank, config.expert_alignment
    ends = ends.to(torch.int64)
    prev = torch.cat((ends.new_zeros(1), ends[:-1]))
    starts = (prev + align - 1) // align * align
    pos = torch.arange(recv_x.shape[0], device=recv_x.device)[:, None]
    belongs = (pos >= starts[None, :]) & (pos < ends[None, :])
    factors = torch.arange(el, device=recv_x.device, dtype=torch.float32) + ffn_rank * el + 1
    factor = (belongs.float() * factors).sum(dim=1)
    out = dequantize(recv_x, recv_scale) * recv_weights[:, None] * factor[:, None]
    return torch.where(belongs.any(dim=1)[:, None], out, torch.zeros_like(out)).to(torch.bfloat16)


def expected_combine(config: Config, src: SourceBatch, expert_fn=None, stages: str = "two_stage") -> torch.Tensor:
    """BF16 [T, H]: what ``source_collect`` must return for one source.

    ``expert_fn(e, x_fp32) -> fp32`` defaults to the synthetic expert ``(e + 1) * x``.
    ``stages``: "two_stage" (what the transport does) or "single_stage" (one fp32 sum over all
    K rows), which differs by at most one BF16 rounding per FFN rank.
    """
    ids = legal_ids(src.ids, config.num_experts).cpu()
    xf = dequantize(src.x.cpu(), src.x_scale.cpu() if src.x_scale is not None else None)
    w = src.weights.cpu().float()
    T, K = ids.shape
    el = config.experts_per_rank
    out = torch.zeros((T, config.hidden_size), dtype=torch.float32)
    per_rank = [torch.zeros_like(out) for _ in range(config.ffn_ranks)]
    n_rank = torch.zeros((config.ffn_ranks, T), dtype=torch.int64)
    for k in range(K):
        e = ids[:, k]
        sel = e >= 0
        if not sel.any():
            continue
        ex = e.clamp(min=0)
        if expert_fn is None:
            # same operation order as synthetic_expert_rows: (x * weight) * (e + 1)
            y = xf * w[:, k][:, None] * (ex + 1).float()[:, None]
        else:
            y = torch.zeros_like(xf)
            for ee in torch.unique(ex[sel]).tolist():
                m = sel & (ex == ee)
                y[m] = expert_fn(int(ee), xf[m]) * w[m, k][:, None]
        row = y.to(torch.bfloat16).float()   # the caller replies in BF16
        row = torch.where(sel[:, None], row, torch.zeros_like(row))
        if stages == "single_stage":
            out += row
        else:
            f = ex // el
            for ff in range(config.ffn_ranks):
                m = sel & (f == ff)
                per_rank[ff][m] += row[m]
                n_rank[ff][m] += 1
    if stages == "single_stage":
        return out.to(torch.bfloat16)
    for ff in range(config.ffn_ranks):
        out += per_rank[ff].to(torch.bfloat16).float()
    return out.to(torch.bfloat16)


def receive_rows_exact(config: Config, ffn_rank: int, all_ids: list[torch.Tensor]) -> int:
    el = config.experts_per_rank
    lo = ffn_rank * el
    total = 0
    counts = sum(expert_counts(legal_ids(i, config.num_experts).cpu(), config.num_experts)[lo : lo + el] for i in all_ids)
    for c in counts.tolist():
        total += align_up(int(c), config.expert_alignment)
    return total
