"""tcgen05 grouped GEMM against an fp32 torch reference of the same operation."""

import pytest
import torch

from afdep_b200.ops import grouped_gemm as gg

pytestmark = pytest.mark.gpu


def _segments(counts, alignment):
    ends, run = [], 0
    for c in counts:
        run = (run + alignment - 1) // alignment * alignment
        run += c
        ends.append(run)
    rows = (run + alignment - 1) // alignment * alignment
    return torch.tensor(ends, dtype=torch.int32), rows


TILES = ["wide", "swapped"]     # 128 rows x 256 columns per tile, or 128 weight rows x 64 tokens


@pytest.mark.parametrize("tile", TILES)
@pytest.mark.parametrize("counts,N,K", [([128], 128, 64 * 2), ([100, 0, 300, 128], 256, 512), ([37, 260, 129, 5, 640, 1], 512, 1024)])
def test_bf16_grouped_gemm(counts, N, K, tile):
    torch.manual_seed(0)
    ends, rows = _segments(counts, 128)
    a = (torch.randn(rows, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(len(counts), N, K, device="cuda") * 0.05).bfloat16()
    out = torch.full((rows, N), 7.0, device="cuda", dtype=torch.bfloat16)
    gg.grouped_gemm(a, w, ends.cuda(), 128, out=out, tile=tile)
    torch.cuda.synchronize()
    ref = gg.reference_grouped_gemm(a, w, ends, 128)
    starts = gg.segment_starts(ends, 128).tolist()
    for e, (s, t) in enumerate(zip(starts, ends.tolist())):
        torch.testing.assert_close(out[s:t].float(), ref[s:t], rtol=2e-2, atol=2e-2)
    # rows outside every segment are untouched
    mask = torch.ones(rows, dtype=torch.bool)
    for s, t in zip(starts, ends.tolist()):
        mask[s:t] = False
    assert (out[mask.cuda()] == 7.0).all()


@pytest.mark.parametrize("tile", TILES)
def test_bf16_swiglu_and_row_scale(tile):
    torch.manual_seed(1)
    counts, I, K = [200, 77, 0, 130], 256, 512
    ends, rows = _segments(counts, 128)
    a = (torch.randn(rows, K, device="cuda") * 0.5).bfloat16()
    wg = (torch.randn(len(counts), I, K, device="cuda") * 0.05).bfloat16()
    wu = (torch.randn(len(counts), I, K, device="cuda") * 0.05).bfloat16()
    w = gg.interleave_gate_up(wg, wu)
    scale = torch.rand(rows, device="cuda") + 0.5
    out = gg.grouped_gemm(a, w, ends.cuda(), 128, swiglu=True, row_scale=scale, tile=tile)
    torch.cuda.synchronize()
    ref = gg.reference_grouped_gemm(a, w, ends, 128, swiglu=True, row_scale=scale)
    # direct statement of the same thing from the un-interleaved matrices
    starts = gg.segment_starts(ends, 128).tolist()
    for e, (s, t) in enumerate(zip(starts, ends.tolist())):
        if t <= s:
            continue
        x = a[s:t].float()
        direct = torch.nn.functional.silu(x @ wg[e].float().T) * (x @ wu[e].float().T) * scale[s:t, None]
        torch.testing.assert_close(ref[s:t], direct, rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(out[s:t].float(), ref[s:t], rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("tile", TILES)
@pytest.mark.parametrize("swiglu", [False, True])
def test_fp8_block_scaled_grouped_gemm(swiglu, tile):
    torch.manual_seed(2)
    counts, N, K = [150, 0, 128, 300], 256, 1024
    ends, rows = _segments(counts, 128)
    x = torch.randn(rows, K, device="cuda")
    wf = torch.randn(len(counts), N, K, device="cuda") * 0.02
    a, a_scale = gg.quantize_rows_fp8(x)
    w, w_scale = gg.quantize_weight_blocks_fp8(wf)
    scale = torch.rand(rows, device="cuda") + 0.5
    # a column-major scale view, the layout worker_receive can return
    a_scale_cm = a_scale.t().contiguous().t()
    out = gg.grouped_gemm(a, w, ends.cuda(), 128, swiglu=swiglu, row_scale=scale, a_scale=a_scale_cm, w_scale=w_scale, tile=tile)
    torch.cuda.synchronize()
    ref = gg.reference_grouped_gemm(a, w, ends, 128, swiglu=swiglu, row_scale=scale, a_scale=a_scale, w_scale=w_scale)
    starts = gg.segment_starts(ends, 128).tolist()
    for s, t in zip(starts, ends.tolist()):
        torch.testing.assert_close(out[s:t].float(), ref[s:t], rtol=2e-2, atol=2e-2)


def test_fp8_swiglu_with_quantised_output_feeds_an_fp8_down_projection():
    """The SwiGLU epilogue can emit e4m3 rows with per-row, per-128-column scales; they must
    dequantise to the fp32 SwiGLU output within e4m3 rounding, and a second FP8 GEMM on them
    must match the reference evaluated on the same quantised rows."""
    torch.manual_seed(4)
    counts, I, K, H2 = [140, 0, 128, 260], 512, 1024, 384
    ends, rows = _segments(counts, 128)
    x = torch.randn(rows, K, device="cuda")
    a, a_scale = gg.quantize_rows_fp8(x)
    wg = torch.randn(len(counts), I, K, device="cuda") * 0.03
    wu = torch.randn(len(counts), I, K, device="cuda") * 0.03
    w, w_scale = gg.quantize_weight_blocks_fp8(gg.interleave_gate_up(wg, wu))
    h_q, h_scale = gg.grouped_gemm(a, w, ends.cuda(), 128, swiglu=True, a_scale=a_scale, w_scale=w_scale, quantize_out=True)
    torch.cuda.synchronize()
    assert h_q.dtype == torch.float8_e4m3fn and h_q.shape == (rows, I) and h_scale.shape == (rows, I // 128)
    ref = gg.reference_grouped_gemm(a, w, ends, 128, swiglu=True, a_scale=a_scale, w_scale=w_scale)
    starts = gg.segment_starts(ends, 128).tolist()
    for s0, t0 in zip(starts, ends.tolist()):
        if t0 <= s0:
            continue
        r = ref[s0:t0].view(t0 - s0, I // 128, 128)
        sc = h_scale[s0:t0]
        torch.testing.assert_close(sc, r.abs().amax(dim=2).clamp_min(1e-12) / 448.0, rtol=2e-2, atol=1e-9)
        dq = h_q[s0:t0].float().view(t0 - s0, I // 128, 128) * sc[:, :, None]
        bound = r.abs() * 0.09 + sc[:, :, None] * 2.0 ** -8
        assert ((dq - r).abs() <= bound).all()
    # down projection in FP8 on the quantised rows
    wd, wd_scale = gg.quantize_weight_blocks_fp8(torch.randn(len(counts), H2, I, device="cuda") * 0.03)
    rs = torch.rand(rows, device="cuda") + 0.5
    out = gg.grouped_gemm(h_q, wd, ends.cuda(), 128, row_scale=rs, a_scale=h_scale, w_scale=wd_scale)
    torch.cuda.synchronize()
    # rows outside the segments hold unspecified bytes: zero them for the reference
    hq_clean, hs_clean = torch.zeros_like(h_q.float()), torch.ones_like(h_scale)
    for s0, t0 in zip(starts, ends.tolist()):
        hq_clean[s0:t0], hs_clean[s0:t0] = h_q[s0:t0].float(), h_scale[s0:t0]
    ref2 = gg.reference_grouped_gemm(hq_clean.to(torch.float8_e4m3fn), wd, ends, 128, row_scale=rs, a_scale=hs_clean, w_scale=wd_scale)
    for s0, t0 in zip(starts, ends.tolist()):
        torch.testing.assert_close(out[s0:t0].float(), ref2[s0:t0], rtol=2e-2, atol=2e-3)


def test_fp8_row_quantiser_matches_torch():
    torch.manual_seed(3)
    x = (torch.randn(300, 1024, device="cuda") * 3).bfloat16()
    x[7] = 0                                         # an all-zero group must not divide by zero
    limit = torch.tensor([257], dtype=torch.int32, device="cuda")
    q, s = gg.quantize_rows_fp8_cuda(x, limit)
    _, sr = gg.quantize_rows_fp8(x)
    torch.cuda.synchronize()
    torch.testing.assert_close(s[:257], sr[:257], rtol=1e-5, atol=0)
    # every value comes back within half an e4m3 step (2^-4 relative, or the group's smallest step)
    xf = x[:257].float().view(257, -1, 128)
    dq = q[:257].float().view(257, -1, 128) * s[:257, :, None]
    bound = xf.abs() * 0.0625 + s[:257, :, None] * 2.0 ** -9 + 1e-30
    assert ((dq - xf).abs() <= bound).all()
    assert (dq[7] == 0).all()


def test_unknown_tile_is_rejected():
    with pytest.raises(ValueError):
        gg.grouped_gemm(torch.zeros(1), torch.zeros(1), torch.zeros(1), 128, tile="tall")
