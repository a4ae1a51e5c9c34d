"""Grouped expert GEMMs on tcgen05 tensor cores, and the plain-torch reference they are tested against.

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
                 quantize_out: bool = False):
    """The promoting kernel: BF16, or e4m3 with arbitrary fp32 block scales (every 128-deep K
    block is scaled in registers on its way out of tensor memory).

    ``quantize_out=True`` (FP8 operands with ``swiglu``): the epilogue quantises the SwiGLU output
    and returns ``(e4m3 [rows, N/2], fp32 scales [rows, N/256])`` instead of BF16, in the per-row,
    per-128-column format the FP8 GEMM takes as its ``a`` operand."""
    from .._native import load_native

    return load_native().grouped_gemm(a, w, ends, int(alignment), bool(swiglu), row_scale, a_scale, w_scale, out, int(ctas), bool(quantize_out))


def expert_gemm(a, w, ends, alignment: int, *, swiglu: bool = False, row_scale=None, a_scale=None, w_scale=None, out=None, ctas: int = 0,
                quantize_out: bool = False, row_index=None, a_scale_offset: int = -1, a_scale_packed: bool = False):
    """The self-feeding kernel: BF16, or e4m3 whose fp32 block scales are **powers of two**
    (``quantize_*(..., pow2=True)``).  The tensor core applies the scales itself
    (``tcgen05.mma ... block_scale``), so the whole K extent accumulates in tensor memory.

    ``row_index`` (int32 ``[rows]``) switches to the gathered form: row ``r`` of the product's row
    space is read from ``a[row_index[r]]`` (negative: a row of zeros), ``a`` being any contiguous
    2-D tensor whose rows start with the K operand elements -- for instance the wire records of an
    exchange, viewed as ``uint8 [records, record_bytes]`` with each record's fp32 scales at byte
    offset ``a_scale_offset``.  ``quantize_out`` returns e4m3 with power-of-two scales.

    The scales of ``a`` may also come as exponent bytes packed four to an int32 word
    (``utils.scales.pack_ue8m0x4``): pass ``a_scale`` as int32 ``[rows, ceil(K/512)]`` (any strides), or
    ``a_scale_packed=True`` for words inside gathered records; they reach tensor memory unconverted."""
    from .._native import load_native

    return load_native().expert_gemm(a, w, ends, int(alignment), bool(swiglu), row_scale, a_scale, w_scale, out, int(ctas), bool(quantize_out),
                                     row_index, int(a_scale_offset), bool(a_scale_packed))


def gemm_check(device: int | None = None) -> bool:
    """True (once) if an expert GEMM on ``device`` abandoned a bounded wait since the last check."""
    from .._native import load_native

    return bool(load_native().gemm_check(torch.cuda.current_device() if device is None else int(device)))


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


from ..utils.scales import pack_ue8m0x4, unpack_ue8m0x4  # noqa: E402,F401  (re-exported next to the quantisers)


def pow2_ceil(scale: torch.Tensor) -> torch.Tensor:
    """Positive fp32 values rounded up to powers of two (exact: mantissa and exponent are split,
    never a logarithm)."""
    mant, exp = torch.frexp(scale.float())               # scale = mant * 2^exp, mant in [0.5, 1)
    exp = exp - (mant == 0.5).to(exp.dtype)              # already a power of two: keep it
    return torch.ldexp(torch.ones_like(mant), exp)


def quantize_rows_fp8_cuda(x: torch.Tensor, limit: torch.Tensor | None = None, pow2: bool = False):
    """The same quantisation as ``quantize_rows_fp8`` in one CUDA kernel (bf16 input on the GPU).
    ``limit``: optional int32 device tensor; rows at or beyond ``limit[0]`` are left unwritten."""
    from .._native import load_native

    return load_native().quantize_rows_fp8(x, limit, bool(pow2))


def quantize_rows_fp8(x: torch.Tensor, pow2: bool = False):
    """e4m3 rows with one fp32 scale per row and 128 columns (amax / 448, optionally rounded up
    to a power of two)."""
    rows, K = x.shape
    g = x.float().view(rows, K // 128, 128)
    scale = (g.abs().amax(dim=2).double().clamp_min(1e-12) / 448.0).float()     # true division (a scalar divisor may be turned into a reciprocal)
    if pow2:
        scale = pow2_ceil(scale)
    return (g / scale[:, :, None]).reshape(rows, K).to(torch.float8_e4m3fn), scale


def quantize_weight_blocks_fp8(w: torch.Tensor, pow2: bool = False):
    """e4m3 weights with one fp32 scale per 128 x 128 block: ([E, N, K] e4m3, [E, N/128, K/128])."""
    E, N, K = w.shape
    g = w.float().view(E, N // 128, 128, K // 128, 128)
    scale = (g.abs().amax(dim=(2, 4)).double().clamp_min(1e-12) / 448.0).float()
    if pow2:
        scale = pow2_ceil(scale)
    q = (g / scale[:, :, None, :, None]).reshape(E, N, K).to(torch.float8_e4m3fn)
    return q, scale.contiguous()
