"""CPU checks of the plain-torch quantisers the GPU kernels are tested against, and of the small
host-side pieces added beside them (power-of-two scale rounding, the event hand-back object)."""

import pytest
import torch

from afdep_b200.ops import grouped_gemm as gg
from afdep_b200.utils import synthetic


def test_pow2_ceil_is_exact_and_never_rounds_down():
    x = torch.tensor([2.0 ** -6, 2.0 ** -6 * (1 + 2.0 ** -20), 0.5, 0.75, 1.0, 3.0, 448.0, 1e-12, 7.0 / 448.0])
    for fn in (gg.pow2_ceil, synthetic.pow2_ceil):
        y = fn(x)
        assert torch.equal(torch.log2(y), torch.round(torch.log2(y)))          # powers of two
        assert bool((y >= x).all()) and bool((y < 2 * x).all())               # the smallest one not below x
        assert float(y[0]) == 2.0 ** -6 and float(y[1]) == 2.0 ** -5 and float(y[8]) == 2.0 ** -6


def test_row_and_block_quantisers_round_trip_within_e4m3_precision():
    torch.manual_seed(0)
    x = torch.randn(37, 512) * 3
    x[5] = 0
    for pow2 in (False, True):
        q, s = gg.quantize_rows_fp8(x, pow2)
        assert q.dtype == torch.float8_e4m3fn and s.shape == (37, 4)
        dq = q.float().view(37, 4, 128) * s[:, :, None]
        assert bool(((dq - x.view(37, 4, 128)).abs() <= x.view(37, 4, 128).abs() * 0.0625 + s[:, :, None] * 2.0 ** -9 + 1e-30).all())
        assert bool((q.float().abs() <= 448).all()) and bool((dq[5] == 0).all())
        if pow2:
            assert torch.equal(torch.log2(s), torch.round(torch.log2(s)))
        w = torch.randn(2, 256, 384) * 0.02
        wq, ws = gg.quantize_weight_blocks_fp8(w, pow2)
        assert ws.shape == (2, 2, 3)
        wd = (wq.float().view(2, 2, 128, 3, 128) * ws.view(2, 2, 1, 3, 1)).reshape(2, 256, 384)
        assert float((wd - w).abs().max()) <= float(w.abs().max()) * 0.0625 + 1e-6
        sq, ss = synthetic.quantize_fp8(x, pow2)
        assert torch.equal(sq.view(torch.uint8), q.view(torch.uint8)) and torch.equal(ss, s)     # the two statements agree


def test_reference_grouped_gemm_applies_block_scales_and_swiglu():
    torch.manual_seed(1)
    ends = torch.tensor([100, 128 + 60], dtype=torch.int32)
    a = torch.randn(256, 256)
    wg, wu = torch.randn(2, 128, 256) * 0.05, torch.randn(2, 128, 256) * 0.05
    w = gg.interleave_gate_up(wg, wu)
    out = gg.reference_grouped_gemm(a, w, ends, 128, swiglu=True)
    want0 = torch.nn.functional.silu(a[:100] @ wg[0].T) * (a[:100] @ wu[0].T)
    want1 = torch.nn.functional.silu(a[128:188] @ wg[1].T) * (a[128:188] @ wu[1].T)
    torch.testing.assert_close(out[:100], want0, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(out[128:188], want1, rtol=1e-4, atol=1e-4)
    assert not out[100:128].any() and not out[188:].any()


def test_event_handle_without_a_stream_is_a_no_op():
    from afdep_b200.parallel.native_transport import EventHandle

    h = EventHandle(torch, None, (torch.zeros(1),))
    assert h.query() is True
    h.current_stream_wait()
    h.synchronize()
    assert h._keep_alive == ()


def test_ue8m0x4_pack_round_trip_and_refusals():
    """Exponent bytes four to an int32 word: every fp32 power of two survives, padding bytes carry
    the exponent of 1.0, strided inputs are read as they are, anything else is refused."""
    from afdep_b200.utils.scales import UE8M0_ONE, pack_ue8m0x4, unpack_ue8m0x4

    g = torch.Generator().manual_seed(5)
    scale = torch.ldexp(torch.ones(9, 7), torch.randint(-126, 128, (9, 7), generator=g))
    scale[0, 3], scale[1, 0] = 2.0 ** 127, 2.0 ** -126        # both ends of the range; the first sets a word's sign bit
    words = pack_ue8m0x4(scale)
    assert words.dtype == torch.int32 and words.shape == (9, 2)
    assert torch.equal(unpack_ue8m0x4(words, 7), scale)
    assert torch.equal((words[:, 1].long() >> 24) & 0xFF, torch.full((9,), UE8M0_ONE))      # the eighth byte is padding
    col_major = words.t().contiguous().t()
    assert not col_major.is_contiguous() and torch.equal(unpack_ue8m0x4(col_major, 7), scale)
    for bad in (torch.tensor([[3.0]]), torch.tensor([[0.0]]), torch.tensor([[-2.0]]), torch.tensor([[1e-40]])):
        with pytest.raises(ValueError, match="power-of-two"):
            pack_ue8m0x4(bad)


def test_config_scale_format():
    from afdep_b200 import Config

    c = Config(16, 7168, 8, 2, 2, 2, payload="fp8", scale_format="ue8m0x4")
    assert c.scale_packed and c.scale_groups == 14                 # 56 scales, four to a word
    assert Config(16, 768, 8, 2, 2, 2, payload="fp8", scale_format="ue8m0x4").scale_groups == 2     # 6 scales: padded
    assert Config(16, 7168, 8, 2, 2, 2, payload="fp8").scale_groups == 56
    with pytest.raises(ValueError, match="scale_format"):
        Config(16, 512, 8, 2, 2, 2, payload="fp8", scale_format="e8m0")
    with pytest.raises(ValueError, match="FP8 payloads only"):
        Config(16, 512, 8, 2, 2, 2, scale_format="ue8m0x4")
