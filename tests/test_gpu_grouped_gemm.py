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


def _bf16_op(kernel):
    return gg.grouped_gemm if kernel == "promoting" else gg.expert_gemm


KERNELS = ["promoting", "selffeeding"]     # grouped_gemm.cu / expert_gemm.cu


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("counts,N,K", [([128], 128, 64 * 2), ([100, 0, 300, 128], 256, 512), ([37, 260, 129, 5, 640, 1], 512, 1024), ([128, 128], 4096, 7168)])
def test_bf16_grouped_gemm(counts, N, K, kernel):
    torch.manual_seed(0)
    ends, rows = _segments(counts, 128)
    a = (torch.randn(rows, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(len(counts), N, K, device="cuda") * 0.05).bfloat16()
    out = torch.full((rows, N), 7.0, device="cuda", dtype=torch.bfloat16)
    _bf16_op(kernel)(a, w, ends.cuda(), 128, out=out)
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


@pytest.mark.parametrize("kernel", KERNELS)
def test_bf16_swiglu_and_row_scale(kernel):
    torch.manual_seed(1)
    counts, I, K = [200, 77, 0, 130], 256, 512
    ends, rows = _segments(counts, 128)
    a = (torch.randn(rows, K, device="cuda") * 0.5).bfloat16()
    wg = (torch.randn(len(counts), I, K, device="cuda") * 0.05).bfloat16()
    wu = (torch.randn(len(counts), I, K, device="cuda") * 0.05).bfloat16()
    w = gg.interleave_gate_up(wg, wu)
    scale = torch.rand(rows, device="cuda") + 0.5
    out = _bf16_op(kernel)(a, w, ends.cuda(), 128, swiglu=True, row_scale=scale)
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


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("shape", [([150, 0, 128, 300], 256, 1024), ([128, 128], 4096, 7168), ([90, 200], 384, 640)])
@pytest.mark.parametrize("swiglu", [False, True])
def test_fp8_block_scaled_grouped_gemm(swiglu, shape, kernel):
    """fp32 block scales through the promoting kernel; power-of-two block scales through the
    self-feeding kernel, where the tensor core applies them.  The large case is the gate|up shape
    of the end-to-end benchmark (56 trips round the stage ring, 14 scale groups); the last one has
    a K extent that is not a multiple of four blocks and a half-empty last column tile."""
    torch.manual_seed(2)
    counts, N, K = shape
    if swiglu and N % 256:
        pytest.skip("SwiGLU pairs need whole 64-column groups in every tile half")
    pow2 = kernel == "selffeeding"
    ends, rows = _segments(counts, 128)
    x = torch.randn(rows, K, device="cuda")
    wf = torch.randn(len(counts), N, K, device="cuda") * 0.02
    a, a_scale = gg.quantize_rows_fp8(x, pow2)
    w, w_scale = gg.quantize_weight_blocks_fp8(wf, pow2)
    scale = torch.rand(rows, device="cuda") + 0.5
    # a column-major scale view, the layout worker_receive returns
    a_scale_cm = a_scale.t().contiguous().t()
    op = gg.expert_gemm if pow2 else gg.grouped_gemm
    out = op(a, w, ends.cuda(), 128, swiglu=swiglu, row_scale=scale, a_scale=a_scale_cm, w_scale=w_scale)
    torch.cuda.synchronize()
    ref = gg.reference_grouped_gemm(a, w, ends, 128, swiglu=swiglu, row_scale=scale, a_scale=a_scale, w_scale=w_scale)
    starts = gg.segment_starts(ends, 128).tolist()
    for s, t in zip(starts, ends.tolist()):
        torch.testing.assert_close(out[s:t].float(), ref[s:t], rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("kernel", KERNELS)
def test_fp8_swiglu_with_quantised_output_feeds_an_fp8_down_projection(kernel):
    """The SwiGLU epilogue can emit e4m3 rows with per-row, per-128-column scales; they must
    dequantise to the fp32 SwiGLU output within e4m3 rounding, and a second FP8 GEMM on them
    must match the reference evaluated on the same quantised rows."""
    torch.manual_seed(4)
    pow2 = kernel == "selffeeding"
    op = gg.expert_gemm if pow2 else gg.grouped_gemm
    counts, I, K, H2 = [140, 0, 128, 260], 512, 1024, 384
    ends, rows = _segments(counts, 128)
    x = torch.randn(rows, K, device="cuda")
    a, a_scale = gg.quantize_rows_fp8(x, pow2)
    wg = torch.randn(len(counts), I, K, device="cuda") * 0.03
    wu = torch.randn(len(counts), I, K, device="cuda") * 0.03
    w, w_scale = gg.quantize_weight_blocks_fp8(gg.interleave_gate_up(wg, wu), pow2)
    h_q, h_scale = op(a, w, ends.cuda(), 128, swiglu=True, a_scale=a_scale, w_scale=w_scale, quantize_out=True)
    torch.cuda.synchronize()
    assert h_q.dtype == torch.float8_e4m3fn and h_q.shape == (rows, I) and h_scale.shape == (rows, I // 128)
    ref = gg.reference_grouped_gemm(a, w, ends, 128, swiglu=True, a_scale=a_scale, w_scale=w_scale)
    starts = gg.segment_starts(ends, 128).tolist()
    for s0, t0 in zip(starts, ends.tolist()):
        if t0 <= s0:
            continue
        r = ref[s0:t0].view(t0 - s0, I // 128, 128)
        sc = h_scale[s0:t0]
        want_scale = r.abs().amax(dim=2).clamp_min(1e-12) / 448.0
        if pow2:
            # a power of two at or just above amax / 448 (the kernel's fp32 SwiGLU may differ in the last bits)
            assert bool((torch.log2(sc) == torch.round(torch.log2(sc))).all())
            assert bool((sc >= want_scale * 0.98).all()) and bool((sc <= want_scale * 2.04).all())
        else:
            torch.testing.assert_close(sc, want_scale, rtol=2e-2, atol=1e-9)
        dq = h_q[s0:t0].float().view(t0 - s0, I // 128, 128) * sc[:, :, None]
        bound = r.abs() * 0.09 + sc[:, :, None] * 2.0 ** -8
        assert ((dq - r).abs() <= bound).all()
    # down projection in FP8 on the quantised rows
    wd, wd_scale = gg.quantize_weight_blocks_fp8(torch.randn(len(counts), H2, I, device="cuda") * 0.03, pow2)
    rs = torch.rand(rows, device="cuda") + 0.5
    out = op(h_q, wd, ends.cuda(), 128, row_scale=rs, a_scale=h_scale, w_scale=wd_scale)
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


def test_pow2_row_quantiser_emits_exact_powers_of_two():
    torch.manual_seed(5)
    x = (torch.randn(200, 512, device="cuda") * 2).bfloat16()
    q, s = gg.quantize_rows_fp8_cuda(x, None, True)
    _, sr = gg.quantize_rows_fp8(x, True)
    torch.cuda.synchronize()
    assert torch.equal(s, sr)
    assert bool((torch.log2(s) == torch.round(torch.log2(s))).all())
    dq = q.float().view(200, -1, 128) * s[:, :, None]
    xf = x.float().view(200, -1, 128)
    assert ((dq - xf).abs() <= xf.abs() * 0.0625 + s[:, :, None] * 2.0 ** -9 + 1e-30).all()


@pytest.mark.parametrize("dtype", ["bf16", "fp8"])
def test_gathered_rows_match_the_dense_product(dtype):
    """Rows of A picked by index out of a matrix of "records" (here: rows longer than K, FP8 with
    the row's scales stored behind the payload, as in a wire record).  Negative indices are rows of
    zeros; the result must equal the dense kernel on the materialised rows."""
    torch.manual_seed(6)
    counts, N, K = [70, 0, 200, 129], 512, 1024
    ends, rows = _segments(counts, 128)
    n_rec = 300
    index = torch.randint(0, n_rec, (rows,), dtype=torch.int32)
    index[5] = -1
    index[77] = -1
    if dtype == "bf16":
        records = (torch.randn(n_rec, K + 64, device="cuda") * 0.5).bfloat16()       # 128 bytes of other data behind every row
        w = (torch.randn(len(counts), N, K, device="cuda") * 0.05).bfloat16()
        dense = records[index.clamp_min(0).cuda().long(), :K].contiguous()
        dense[index.cuda() < 0] = 0
        got = gg.expert_gemm(records, w, ends.cuda(), 128, row_index=index.cuda())
        want = gg.expert_gemm(dense, w, ends.cuda(), 128)
        ref = gg.reference_grouped_gemm(dense, w, ends, 128)
    else:
        x = torch.randn(n_rec, K, device="cuda")
        q, sc = gg.quantize_rows_fp8(x, True)
        rec_bytes = K + (K // 128) * 4 + 96
        records = torch.zeros(n_rec, rec_bytes, dtype=torch.uint8, device="cuda")
        records[:, :K] = q.view(torch.uint8)
        records[:, K : K + (K // 128) * 4] = sc.contiguous().view(torch.uint8).view(n_rec, -1)
        w, w_scale = gg.quantize_weight_blocks_fp8(torch.randn(len(counts), N, K, device="cuda") * 0.02, True)
        sel = index.clamp_min(0).cuda().long()
        dense, dense_scale = q[sel].contiguous(), sc[sel].contiguous()
        dense.view(torch.uint8)[index.cuda() < 0] = 0
        dense_scale[index.cuda() < 0] = 1.0
        got = gg.expert_gemm(records, w, ends.cuda(), 128, w_scale=w_scale, row_index=index.cuda(), a_scale_offset=K)
        want = gg.expert_gemm(dense, w, ends.cuda(), 128, a_scale=dense_scale, w_scale=w_scale)
        ref = gg.reference_grouped_gemm(dense, w, ends, 128, a_scale=dense_scale, w_scale=w_scale)
        # the same scales as exponent bytes packed four to a word: dense (row- and column-major words)
        # and inside the records
        words = gg.pack_ue8m0x4(dense_scale)
        packed = [gg.expert_gemm(dense, w, ends.cuda(), 128, a_scale=words, w_scale=w_scale),
                  gg.expert_gemm(dense, w, ends.cuda(), 128, a_scale=words.t().contiguous().t(), w_scale=w_scale)]
        rec_words = gg.pack_ue8m0x4(sc)
        records2 = torch.zeros(n_rec, K + 128, dtype=torch.uint8, device="cuda")
        records2[:, :K] = q.view(torch.uint8)
        records2[:, K : K + rec_words.shape[1] * 4] = rec_words.contiguous().view(torch.uint8).view(n_rec, -1)
        packed.append(gg.expert_gemm(records2, w, ends.cuda(), 128, w_scale=w_scale, row_index=index.cuda(), a_scale_offset=K, a_scale_packed=True))
    torch.cuda.synchronize()
    starts = gg.segment_starts(ends, 128).tolist()
    for s0, t0 in zip(starts, ends.tolist()):
        assert torch.equal(got[s0:t0], want[s0:t0])
        if dtype == "fp8":
            for other in packed:
                assert torch.equal(other[s0:t0], want[s0:t0])
        torch.testing.assert_close(got[s0:t0].float(), ref[s0:t0], rtol=2e-2, atol=2e-2)
    assert not gg.gemm_check()
