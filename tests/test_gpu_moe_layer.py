"""End-to-end AFD MoE layer on one GPU (loopback world): exchange + tcgen05 expert MLP."""

import pytest
import torch

from afdep_b200 import Config
from afdep_b200.models.moe_layer import ExpertWeights, reference_experts, run_experts
from afdep_b200.ops import grouped_gemm as gg
from afdep_b200.utils import synthetic

pytestmark = pytest.mark.gpu


def _dequant_blocks(w, scale):
    if scale is None:
        return w.float()
    E, N, K = w.shape
    return (w.float().view(E, N // 128, 128, K // 128, 128) * scale.view(E, N // 128, 1, K // 128, 1)).reshape(E, N, K)


CASES = [
    # payload, expert storage, down projection, FP8 scale format, fused receive -> experts -> reply
    ("bf16", "bf16", "bf16", "fp32", False),
    ("fp8", "fp8", "fp8", "fp32", False),
    ("bf16", "fp8", "fp8", "fp32", False),
    ("fp8", "fp8", "bf16", "fp32", False),
    ("fp8", "fp8", "fp8", "pow2", False),
    ("bf16", "fp8", "fp8", "pow2", False),
    ("bf16", "bf16", "bf16", "fp32", True),
    ("fp8", "fp8", "fp8", "pow2", True),
]


@pytest.mark.parametrize("payload,mode,down,scale_format,fused", CASES)
def test_moe_layer_matches_dense_reference(payload, mode, down, scale_format, fused):
    from afdep_b200.parallel.loopback import LoopbackWorld

    hidden, inter, experts, top_k, ffn, attn, tokens = 512, 256, 8, 2, 2, 2, 96
    pow2 = scale_format == "pow2"
    cfg = Config(tokens, hidden, experts, top_k, ffn, attn, expert_alignment=128, payload=payload)
    world = LoopbackWorld(cfg, gpu_timeout_s=5.0)
    try:
        el = cfg.experts_per_rank
        weights = [ExpertWeights.random(el, hidden, inter, mode=mode, down=down, seed=10 + f, scale_format=scale_format) for f in range(ffn)]
        batches = [synthetic.random_batch(cfg, tokens - 7 * a, seed=a, pow2_scales=pow2) for a in range(attn)]
        dev = [tuple(None if t is None else t.cuda() for t in b) for b in batches]

        def expert(i, rec):
            return run_experts(rec, weights[i], cfg.expert_alignment)

        outs, received = world.exchange(dev, expert)
        torch.cuda.synchronize()
        if fused:
            # the same exchange again, this time with the experts reading the wire records directly
            unfused_outs = outs
            unfused_rows = [run_experts(rec, weights[i], cfg.expert_alignment) for i, rec in enumerate(received)]
            for buf, (x, ids, w, scale) in zip(world.attention, dev):
                buf.source_dispatch(x, ids, w, scale, bucket=tokens)
            served = [buf.worker_serve_fused(weights[i], bucket=tokens) for i, buf in enumerate(world.ffn)]
            outs = [buf.source_collect() for buf in world.attention]
            torch.cuda.synchronize()
            for i, ((res, rows), rec) in enumerate(zip(served, received)):
                assert res.recv_x is None and torch.equal(res.recv_count_psum, rec.recv_count_psum)
                ends = rec.recv_count_psum.cpu().tolist()
                start = 0
                for end in ends:
                    start = (start + 127) // 128 * 128
                    assert torch.equal(res.recv_topk_weights[start:end], rec.recv_topk_weights[start:end])
                    assert torch.equal(res.handle.recv_src_metadata[start:end], rec.handle.recv_src_metadata[start:end])
                    torch.testing.assert_close(rows[start:end].float(), unfused_rows[i][start:end].float(), rtol=2e-2, atol=1e-3)
                    start = end
            for o, u in zip(outs, unfused_outs):
                torch.testing.assert_close(o.float(), u.float(), rtol=2e-2, atol=2e-3)
        for b in world.buffers:
            b.check()
        assert not gg.gemm_check()
        # the kernels' rows against the fp32 reference of the same MLP on the same received rows
        for i, rec in enumerate(received):
            got = run_experts(rec, weights[i], cfg.expert_alignment).float()
            want = reference_experts(rec, weights[i], cfg.expert_alignment).float()
            ends = rec.recv_count_psum.cpu().tolist()
            start = 0
            for e, end in enumerate(ends):
                start = (start + 127) // 128 * 128
                torch.testing.assert_close(got[start:end], want[start:end], rtol=3e-2, atol=2e-3)
                start = end
        # and the collected tokens against a dense per-token evaluation
        for a, out in enumerate(outs):
            x, ids, w, scale = dev[a]
            xf = x.float() if scale is None else (x.float().view(x.shape[0], -1, 128) * scale[:, :, None]).reshape(x.shape[0], -1)
            if scale is None and mode == "fp8":      # BF16 rows are quantised on the FFN rank before they meet FP8 weights
                xq, xs = gg.quantize_rows_fp8(xf, pow2)
                xf = (xq.float().view(xf.shape[0], -1, 128) * xs[:, :, None]).reshape(xf.shape)
            want = torch.zeros_like(xf)
            for f in range(ffn):
                wt = weights[f]
                gu = _dequant_blocks(wt.w_gate_up, wt.w_gate_up_scale)
                wd = _dequant_blocks(wt.w_down, wt.w_down_scale)
                for le in range(el):
                    e = f * el + le
                    sel = ids == e
                    tok = sel.any(dim=1)
                    if not tok.any():
                        continue
                    y = xf[tok] @ gu[le].T
                    y = y.view(y.shape[0], -1, 2, 32)
                    h = (torch.nn.functional.silu(y[:, :, 0]) * y[:, :, 1]).reshape(y.shape[0], -1)
                    if wt.w_down_scale is not None:      # the kernels quantise the SwiGLU output for an FP8 down projection
                        hq, hs = gg.quantize_rows_fp8(h, pow2)
                        h = (hq.float().view(h.shape[0], -1, 128) * hs[:, :, None]).reshape(h.shape)
                    else:
                        h = h.to(torch.bfloat16).float()
                    o = h @ wd[le].T
                    want[tok] += o * (w * sel)[tok].sum(dim=1, keepdim=True)
            # e4m3 intermediates: a value that sits on a rounding boundary may land on either side in
            # the kernel and in this restatement, so bound the error as a whole and element by element
            assert float((out.float() - want).norm() / want.norm()) < 0.03
            torch.testing.assert_close(out.float(), want, rtol=5e-2, atol=5e-3 if weights[0].w_down_scale is None else 1.2e-2)
    finally:
        world.close()


def test_packed_scales_feed_the_experts_like_fp32_scales():
    """The same FP8 rows dispatched with fp32 power-of-two scales and with the scales packed as
    exponent bytes give bit-identical layer outputs, through the separate calls (the words go to
    the block-scaled GEMM as they are) and through the fused path (which reads them out of the records)."""
    from afdep_b200.parallel.loopback import LoopbackWorld

    hidden, inter, experts, top_k, ffn, attn, tokens = 512, 256, 8, 2, 2, 2, 80
    outs = {}
    for fmt in ("fp32", "ue8m0x4"):
        cfg = Config(tokens, hidden, experts, top_k, ffn, attn, expert_alignment=128, payload="fp8", scale_format=fmt)
        world = LoopbackWorld(cfg, gpu_timeout_s=5.0)
        try:
            weights = [ExpertWeights.random(cfg.experts_per_rank, hidden, inter, mode="fp8", down="fp8", seed=10 + f, scale_format="pow2")
                       for f in range(ffn)]
            batches = [synthetic.random_batch(cfg, tokens - 7 * a, seed=a, pow2_scales=True) for a in range(attn)]
            assert all(b[3].dtype == (torch.int32 if fmt == "ue8m0x4" else torch.float32) for b in batches)
            dev = [tuple(None if t is None else t.cuda() for t in b) for b in batches]
            out, _ = world.exchange(dev, lambda i, rec: run_experts(rec, weights[i], cfg.expert_alignment))
            torch.cuda.synchronize()
            for b in world.buffers:
                b.check()
            outs[fmt] = [o.clone() for o in out]
            for buf, (x, ids, w, scale) in zip(world.attention, dev):
                buf.source_dispatch(x, ids, w, scale, bucket=tokens)
            for i, buf in enumerate(world.ffn):
                buf.worker_serve_fused(weights[i], bucket=tokens)
            outs[fmt + "/fused"] = [buf.source_collect().clone() for buf in world.attention]
            torch.cuda.synchronize()
            for b in world.buffers:
                b.check()
        finally:
            world.close()
    assert not gg.gemm_check()
    for k, a in enumerate(outs["fp32"]):
        assert bool(a.float().abs().sum() > 0)
        for other in ("ue8m0x4", "fp32/fused", "ue8m0x4/fused"):
            assert torch.equal(a, outs[other][k]), other
