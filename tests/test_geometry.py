"""Heap layout and launch shapes are pure functions of the configuration: check, without a GPU,
the alignment rules the bulk copies depend on (16-byte addresses and sizes), that the regions of a
heap do not overlap and are large enough, and that every launch fits an SM's shared memory."""

from hypothesis import given, settings
from hypothesis import strategies as st

from afdep_b200._native import load_native

MAX_SMEM = 227 * 1024


@st.composite
def configs(draw):
    ffn = draw(st.integers(1, 4))
    attn = draw(st.integers(1, 8 - ffn))
    hidden = 256 * draw(st.integers(1, 32))
    experts_local = draw(st.sampled_from([1, 2, 4, 8, 32, 64, 128, 256]))
    top_k = draw(st.integers(1, min(32, experts_local * ffn)))
    capacity = draw(st.sampled_from([1, 8, 100, 128, 2048, 4096]))
    fp8 = draw(st.booleans())
    alignment = draw(st.sampled_from([1, 8, 16, 128]))
    return ffn, attn, hidden, top_k, experts_local * ffn, capacity, fp8, alignment


@settings(max_examples=150, deadline=None)
@given(configs(), st.sampled_from([0, 4096, (4 << 20) + 5]))
def test_heap_regions_are_aligned_disjoint_and_large_enough(cfg, aux):
    ffn, attn, hidden, top_k, experts, capacity, fp8, alignment = cfg
    g = load_native().geometry(ffn, attn, hidden, top_k, experts, capacity, fp8, alignment, aux)
    # records and rows move with bulk copies: 16-byte sizes and offsets, records padded to 128
    assert g["payload_bytes"] == hidden * (1 if fp8 else 2) and g["row_bytes"] == hidden * 2
    assert g["rec_bytes"] % 128 == 0 and g["payload_bytes"] % 16 == 0 and g["meta_off"] % 16 == 0 and g["row_bytes"] % 16 == 0
    assert g["meta_off"] == g["payload_bytes"] + g["scale_bytes"]
    assert g["scale_bytes"] >= (hidden // 128 * 4 if fp8 else 0)
    assert g["meta_bytes"] >= 12 * top_k + 4 and g["meta_off"] + g["meta_bytes"] <= g["rec_bytes"]
    # FFN heap: control words, auxiliary region, counts, flags, staging records, reply rows
    assert g["aux_off"] >= 4 * 8 and g["aux_bytes"] >= aux and g["aux_bytes"] % 4096 == 0
    order = [g["aux_off"] + g["aux_bytes"], g["f_cnt"], g["f_slot_flag"], g["f_stage"], g["f_reply"], g["f_bytes"]]
    assert order == sorted(order) and all(o % 256 == 0 for o in order[1:])
    assert g["f_slot_flag"] - g["f_cnt"] >= attn * g["cnt_stride"] * 8 and g["cnt_stride"] >= g["experts_local"] + 1
    assert g["f_stage"] - g["f_slot_flag"] >= attn * capacity * 4
    assert g["f_reply"] - g["f_stage"] >= attn * capacity * g["rec_bytes"]
    assert g["f_bytes"] - g["f_reply"] >= attn * capacity * g["row_bytes"]
    # attention heap: one reply flag per (FFN rank, slot)
    assert g["a_reply_flag"] == g["aux_off"] + g["aux_bytes"] and g["a_bytes"] - g["a_reply_flag"] >= ffn * capacity * 4


@settings(max_examples=150, deadline=None)
@given(configs(), st.integers(0, 4096))
def test_every_launch_fits_an_sm(cfg, tokens):
    ffn, attn, hidden, top_k, experts, capacity, fp8, alignment = cfg
    tokens = min(tokens, capacity)
    shapes = load_native().launch_shapes(ffn, attn, hidden, top_k, experts, capacity, fp8, alignment, tokens, 27, 54, 148, MAX_SMEM)
    limits = {"dispatch": 27, "collect": 54, "receive": 148, "reply": 2 * 148}
    for name, (ctas, warps, smem) in shapes.items():
        assert 1 <= ctas <= limits[name], name
        assert 1 <= warps <= 16, name
        assert 0 <= smem <= MAX_SMEM, name


def test_known_geometry_of_the_headline_config():
    g = load_native().geometry(2, 2, 4096, 8, 128, 2048, False, 128, 0)
    assert (g["rec_bytes"], g["row_bytes"], g["experts_local"]) == (8320, 8192, 64)      # 8 KB row + 100 B of routing words, padded
    assert g["f_bytes"] < 68 << 20                                                        # registered bytes per FFN rank


def test_packed_scale_words_shrink_the_record():
    """56 fp32 scales take 224 bytes of a 7168-wide FP8 record; as 14 words of four exponent bytes
    they take 64 (padded to 16), and everything behind them moves up."""
    lib = load_native()
    fp32 = lib.geometry(2, 2, 7168, 8, 128, 256, True, 128, 0)
    packed = lib.geometry(2, 2, 7168, 8, 128, 256, True, 128, 0, scale_packs=14)
    assert (fp32["scale_bytes"], packed["scale_bytes"]) == (224, 64)
    assert packed["meta_off"] == 7168 + 64 and packed["meta_off"] % 16 == 0
    assert packed["rec_bytes"] % 128 == 0 and packed["rec_bytes"] <= fp32["rec_bytes"]
