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


@pytest.mark.parametrize("counts,N,K", [([128], 128, 64 * 2), ([100, 0, 300, 128], 256, 512), ([37, 260, 129, 5, 640, 1], 512, 1024)])
def test_bf16_grouped_gemm(counts, N, K):
    torch.manual_seed(0)
    ends, rows = _segments(counts, 128)
    a = (torch.randn(rows, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(len(counts), N, K, device="cuda") * 0.05).bfloat16()
    out = torch.full((rows, N), 7.0, device="cuda", dtype=torch.bfloat16)
    gg.grouped_gemm(a, w, ends.cuda(), 128, out=out)
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


def test_bf16_swiglu_and_row_scale():
    torch.manual_seed(1)
    counts, I, K = [200, 77, 0, 130], 256, 512
    ends, rows = _segments(counts, 128)
    a = (torch.randn(rows, K, device="cuda") * 0.5).bfloat16()
    wg = (torch.randn(len(counts), I, K, device="cuda") * 0.05).bfloat16()
    wu = (torch.randn(len(counts), I, K, device="cuda") * 0.05).bfloat16()
    w = gg.interleave_gate_up(wg, wu)
    scale = torch.rand(rows, device="cuda") + 0.5
    out = gg.grouped_gemm(a, w, ends.cuda(), 128, swiglu=True, row_scale=scale)
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


@pytest.mark.parametrize("swiglu", [False, True])
def test_fp8_block_scaled_grouped_gemm(swiglu):
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
    out = gg.grouped_gemm(a, w, ends.cuda(), 128, swiglu=swiglu, row_scale=scale, a_scale=a_scale_cm, w_scale=w_scale)
    torch.cuda.synchronize()
    ref = gg.reference_grouped_gemm(a, w, ends, 128, swiglu=swiglu, row_scale=scale, a_scale=a_scale, w_scale=w_scale)
    starts = gg.segment_starts(ends, 128).tolist()
    for s, t in zip(starts, ends.tolist()):
        torch.testing.assert_close(out[s:t].float(), ref[s:t], rtol=2e-2, atol=2e-2)


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
