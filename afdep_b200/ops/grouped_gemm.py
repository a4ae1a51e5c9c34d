"""Grouped expert GEMM on tcgen05 tensor cores, and the plain-torch reference it is tested against.

``grouped_gemm(a, w, ends, alignment, ...)`` multiplies the expert-major rows returned by
``worker_receive`` with one weight matrix per local expert:

    out[r] = a[r] @ w[e].T        for rows r of expert e's segment

Operands are BF16, or e4m3 with fp32 block scales (``a_scale [rows, K/128]`` per row and 128
columns, ``w_scale [experts, N/128, K/128]`` per 128 x 128 block).  ``swiglu=True`` expects the
gate and up projections interleaved in blocks of 32 rows of ``w`` (see ``interleave_gate_up``)
and returns ``silu(gate) * up`` with ``N/2`` columns; ``row_scale`` multiplies every output
row (the routing weight); ``quantize_out`` makes the FP8 SwiGLU GEMM emit e4m3 rows with scales,
so a down projection can run in FP8 too.  Rows outside the expert segments are left untouched.
"""

from __future__ import annotations

import torch

GATE_UP_BLOCK = 32   # rows of gate, then rows of up, alternating in the fused gate|up matrix


def grouped_gemm(a, w, ends, alignment: int, *, swiglu: bool = False, row_scale=None, a_scale=None, w_scale=None, out=None, ctas: int = 0,
                 quantize_out: bool = False, tile: str = "wide"):
    """``quantize_out=True`` (FP8 operands with ``swiglu``, wide tile): the epilogue quantises the
    SwiGLU output and returns ``(e4m3 [rows, N/2], fp32 scales [rows, N/256])`` instead of BF16, in
    the per-row, per-128-column format the FP8 GEMM takes as its ``a`` operand.

    ``tile``: ``"wide"`` (128 rows x 256 columns per tile, the default) or ``"swapped"`` (128
    weight rows x 64 tokens: the weights are the MMA's M operand).  Measured on a B200 with 16
    rows per expert, 64 experts, FP8: wide 0.336 ms / swapped 0.423 ms for 4096 x 7168 weights,
    0.195 / 0.264 ms for 7168 x 2048 -- the wide tile already streams the weights at 4.8-5.6 TB/s
    there, so the swapped tile is an alternative kept for narrower batches, not the default."""
    from .._native import load_native

    if tile not in ("wide", "swapped"):
        raise ValueError("tile must be 'wide' or 'swapped'")
    return load_native().grouped_gemm(a, w, ends, int(alignment), bool(swiglu), row_scale, a_scale, w_scale, out, int(ctas), bool(quantize_out),
                                      tile == "swapped")


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """[E, I, K] gate and up -> [E, 2I, K] with alternating 32-row blocks gate, up, gate, up, ..."""
    E, I, K = w_gate.shape
    g = w_gate.reshape(E, I // GATE_UP_BLOCK, GATE_UP_BLOCK, K)
    u = w_up.reshape(E, I // GATE_UP_BLOCK, GATE_UP_BLOCK, K)
    return torch.stack((g, u), dim=2).reshape(E, 2 * I, K).contiguous()


def segment_starts(ends: torch.Tensor, alignment: int) -> torch.Tensor:
    ends = ends.to(torch.int64)
    prev = torch.cat((ends.new_zeros(1), ends[:-1]))
    return (prev + alignment - 1) // alignment * alignment


def reference_grouped_gemm(a, w, ends, alignment, *, swiglu=False, row_scale=None, a_scale=None, w_scale=None, interleaved=True):
    """fp32 reference on dequantised operands; returns fp32 [rows, N or N/2], zero outside segments."""
    rows, K = a.shape
    E, N, _ = w.shape
    af = a.float()
    if a_scale is not None:
        af = (af.view(rows, K // 128, 128) * a_scale.float()[:, :, None]).reshape(rows, K)
    wf = w.float()
    if w_scale is not None:
        wf = (wf.view(E, N // 128, 128, K // 128, 128) * w_scale.float().view(E, N // 128, 1, K // 128, 1)).reshape(E, N, K)
    starts = segment_starts(ends, alignment).tolist()
    out = torch.zeros((rows, N // 2 if swiglu else N), dtype=torch.float32, device=a.device)
    for e, (s, t) in enumerate(zip(starts, ends.tolist())):
        if t <= s:
            continue
        y = af[s:t] @ wf[e].T
        if swiglu:
            y = y.view(t - s, N // (2 * GATE_UP_BLOCK), 2, GATE_UP_BLOCK)
            y = (torch.nn.functional.silu(y[:, :, 0]) * y[:, :, 1]).reshape(t - s, N // 2)
        if row_scale is not None:
            y = y * row_scale[s:t].float()[:, None]
        out[s:t] = y
    return out


def quantize_rows_fp8_cuda(x: torch.Tensor, limit: torch.Tensor | None = None):
    """The same quantisation as ``quantize_rows_fp8`` in one CUDA kernel (bf16 input on the GPU).
    ``limit``: optional int32 device tensor; rows at or beyond ``limit[0]`` are left unwritten."""
    from .._native import load_native

    return load_native().quantize_rows_fp8(x, limit)


def quantize_rows_fp8(x: torch.Tensor):
    """e4m3 rows with one fp32 scale per row and 128 columns (amax / 448)."""
    rows, K = x.shape
    g = x.float().view(rows, K // 128, 128)
    scale = g.abs().amax(dim=2).clamp_min(1e-12) / 448.0
    return (g / scale[:, :, None]).reshape(rows, K).to(torch.float8_e4m3fn), scale


def quantize_weight_blocks_fp8(w: torch.Tensor):
    """e4m3 weights with one fp32 scale per 128 x 128 block: ([E, N, K] e4m3, [E, N/128, K/128])."""
    E, N, K = w.shape
    g = w.float().view(E, N // 128, 128, K // 128, 128)
    scale = g.abs().amax(dim=(2, 4)).clamp_min(1e-12) / 448.0
    q = (g / scale[:, :, None, :, None]).reshape(E, N, K).to(torch.float8_e4m3fn)
    return q, scale.contiguous()
