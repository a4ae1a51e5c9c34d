"""Property checks of the pure-torch oracle (CPU): the two statements of placement agree, and
the conservative receive bound really bounds every legal routing."""

import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from afdep_b200 import Config
from afdep_b200.ops.route_layout import reference_layout
from afdep_b200.utils import oracle, synthetic


@settings(max_examples=40, deadline=None)
@given(
    ffn=st.integers(1, 4),
    attn=st.integers(1, 4),
    el=st.sampled_from([1, 2, 4, 8]),
    top_k=st.integers(1, 6),
    tokens=st.integers(0, 40),
    align=st.sampled_from([1, 4, 16, 128]),
    seed=st.integers(0, 10_000),
)
def test_layout_and_receive_oracle_agree(ffn, attn, el, top_k, tokens, align, seed):
    experts = ffn * el
    top_k = min(top_k, experts)
    cfg = Config(max(tokens, 1), 256, experts, top_k, ffn, attn, expert_alignment=align)
    batches = [synthetic.random_batch(cfg, max(0, tokens - a), seed=seed + a, skip_fraction=0.2) for a in range(attn)]
    sources = [oracle.SourceBatch(*b) for b in batches]
    layouts = [reference_layout(b[1], experts, ffn) for b in batches]
    for f in range(ffn):
        exp = oracle.expected_receive(cfg, f, sources)
        # bound: exact rows never exceed the conservative receive shape
        assert exp.layout.rows_exact <= cfg.receive_rows(cfg.capacity_tokens_per_rank)
        assert exp.layout.rows_exact == oracle.receive_rows_exact(cfg, f, [b[1] for b in batches])
        # placement from the routing layout: row = row_base[source][expert] + pos
        for a, (route_e, pos, slot, counts) in enumerate(layouts):
            assert torch.equal(counts[ffn + f * el : ffn + (f + 1) * el].long(), exp.layout.row_base.new_tensor(
                [int(((route_e >= 0) & (route_e == f * el + j)).sum()) for j in range(el)]))
            t_idx, k_idx = torch.nonzero((route_e >= f * el) & (route_e < (f + 1) * el), as_tuple=True)
            for t, k in zip(t_idx.tolist(), k_idx.tolist()):
                row = int(exp.layout.row_base[a][int(route_e[t, k]) - f * el]) + int(pos[t, k])
                assert exp.valid[row]
                assert exp.recv_src[row].tolist() == [a, t]
                assert float(exp.recv_weights[row]) == float(batches[a][2][t, k])
            # records: one per token with at least one choice on this rank, numbered in token order
            has = ((route_e >= f * el) & (route_e < (f + 1) * el)).any(dim=1)
            assert int(counts[f]) == int(has.sum())
            assert slot[has, f].tolist() == list(range(int(has.sum())))
            assert (slot[~has, f] == -1).all()


@settings(max_examples=25, deadline=None)
@given(tokens=st.integers(1, 30), experts=st.sampled_from([4, 8, 16]), top_k=st.integers(1, 4), seed=st.integers(0, 999))
def test_two_stage_and_single_stage_sums_differ_by_at_most_bf16_rounding(tokens, experts, top_k, seed):
    cfg = Config(tokens, 256, experts, min(top_k, experts), 2, 1, expert_alignment=1)
    x, ids, w, _ = synthetic.random_batch(cfg, tokens, seed=seed)
    two = oracle.expected_combine(cfg, oracle.SourceBatch(x, ids, w), stages="two_stage").float()
    one = oracle.expected_combine(cfg, oracle.SourceBatch(x, ids, w), stages="single_stage").float()
    # one extra BF16 rounding per FFN rank: relative 2^-8 of the partial sums
    bound = 0.02 * (one.abs() + 1.0) + 0.05
    assert ((two - one).abs() <= bound).all()
