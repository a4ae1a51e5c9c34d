"""The CUDA transport on ONE GPU: every rank of a Buffer inside this process.

Each case runs complete exchanges through the public role API and compares what the FFN
ranks receive and what the attention ranks collect with the pure-torch oracle: bit for bit,
because the transport is deterministic and the inputs are exactly representable.
"""

import pytest
import torch

from afdep_b200 import AfdepRouteError, Config
from afdep_b200.utils import oracle, synthetic

pytestmark = pytest.mark.gpu


def to_dev(batch):
    return tuple(None if t is None else t.cuda() for t in batch)


def make_world(cfg, **options):
    from afdep_b200.parallel.loopback import LoopbackWorld

    return LoopbackWorld(cfg, gpu_timeout_s=2.0, **options)


def run_and_check(world, cfg, batches, *, bucket=None, read_host_counts=False, exact=True):
    dev = [to_dev(b) for b in batches]
    sources = [oracle.SourceBatch(b[0], b[1], b[2], b[3]) for b in batches]

    def expert(i, rec):
        return oracle.synthetic_expert_rows(cfg, i, rec.recv_x, rec.recv_scale, rec.recv_topk_weights, rec.recv_count_psum)

    outs, received = world.exchange(dev, expert, bucket=bucket, read_host_counts=read_host_counts)
    torch.cuda.synchronize()
    for b in world.buffers:
        b.check()
    for f, rec in enumerate(received):
        exp = oracle.expected_receive(cfg, f, sources, rows=rec.recv_x.shape[0])
        assert torch.equal(rec.recv_count_psum.cpu().long(), exp.layout.ends), f"ends differ on FFN rank {f}"
        v = exp.valid
        assert torch.equal(rec.recv_x.cpu()[v].float(), exp.recv_x[v].float())
        assert torch.equal(rec.recv_topk_weights.cpu()[v], exp.recv_weights[v])
        assert torch.equal(rec.handle.recv_src_metadata.cpu()[v], exp.recv_src[v])
        if cfg.is_fp8:
            assert torch.equal(rec.recv_scale.cpu()[v], exp.recv_scale[v])
        if read_host_counts:
            assert rec.recv_counts_host == exp.layout.aligned_counts
            assert rec.recv_x.shape[0] == exp.layout.rows_exact
        else:
            assert rec.recv_x.shape[0] == cfg.receive_rows(bucket or cfg.capacity_tokens_per_rank)
    for a, out in enumerate(outs):
        expect = oracle.expected_combine(cfg, sources[a])
        if exact:
            assert torch.equal(out.cpu().float(), expect.float()), f"combine differs on attention rank {a}"
        else:
            torch.testing.assert_close(out.cpu().float(), expect.float(), rtol=2e-2, atol=2e-2)
    return outs, received


@pytest.mark.parametrize("payload", ["bf16", "fp8"])
@pytest.mark.parametrize("ffn,attn,experts,top_k", [(1, 1, 8, 2), (2, 2, 8, 2), (2, 2, 16, 8), (4, 4, 32, 8), (2, 6, 64, 6)])
def test_exact_exchange(payload, ffn, attn, experts, top_k):
    cfg = Config(32, 256, experts, top_k, ffn, attn, expert_alignment=8, payload=payload)
    world = make_world(cfg)
    try:
        for epoch in range(3):
            batches = [synthetic.exact_batch(cfg, 32, a, epoch) for a in range(attn)]
            run_and_check(world, cfg, batches)
    finally:
        world.close()


def test_route_cases_and_host_counts():
    cfg = Config(16, 512, 8, 2, 2, 2, expert_alignment=128)
    world = make_world(cfg)
    n = 16
    cases = [
        dict(active=(n, n)),
        dict(active=(n, n), routing="skew"),
        dict(active=(n, 0)),
        dict(active=(n, n), routing="skip"),
        dict(active=(0, 0)),
        dict(active=(3, 1)),
    ]
    try:
        for host in (False, True):
            for epoch, case in enumerate(cases):
                batches = [
                    synthetic.exact_batch(cfg, n, a, epoch, active=case["active"][a], routing=case.get("routing", "mixed"))
                    for a in range(2)
                ]
                run_and_check(world, cfg, batches, read_host_counts=host)
        # fewer tokens than the bucket, and an empty source
        batches = [synthetic.exact_batch(cfg, 5, 0, 9), synthetic.exact_batch(cfg, 0, 1, 9)]
        run_and_check(world, cfg, batches, bucket=8)
    finally:
        world.close()


@pytest.mark.parametrize("payload", ["bf16", "fp8"])
def test_random_routes_large_hidden(payload):
    cfg = Config(512, 2048, 32, 8, 2, 2, payload=payload)
    world = make_world(cfg)
    try:
        for seed in range(2):
            batches = [synthetic.random_batch(cfg, 512 - 37 * a, 100 * seed + a, skip_fraction=0.1) for a in range(2)]
            run_and_check(world, cfg, batches, exact=True)
        batches = [synthetic.random_batch(cfg, 300, 7 + a, zipf_s=1.1) for a in range(2)]
        run_and_check(world, cfg, batches)
    finally:
        world.close()


def test_strided_scales_and_column_major_output():
    cfg = Config(16, 512, 8, 2, 2, 2, expert_alignment=4, payload="fp8")
    world = make_world(cfg)           # column-major receive scales are the default
    try:
        batches = []
        for a in range(2):
            x, ids, w, scale = synthetic.exact_batch(cfg, 16, a, 3)
            wide = torch.full((16, scale.shape[1] * 2), float("nan"))
            wide[:, ::2] = scale
            batches.append((x, ids, w, wide))
        dev = []
        for x, ids, w, wide in batches:
            dev.append((x.cuda(), ids.cuda(), w.cuda(), wide.cuda()[:, ::2]))
        sources = [oracle.SourceBatch(b[0], b[1], b[2], b[3][:, ::2]) for b in batches]

        def expert(i, rec):
            assert rec.recv_scale.stride(0) == 1 and rec.recv_scale.stride(1) % 4 == 0
            return oracle.synthetic_expert_rows(cfg, i, rec.recv_x, rec.recv_scale, rec.recv_topk_weights, rec.recv_count_psum)

        outs, received = world.exchange(dev, expert)
        torch.cuda.synchronize()
        for a, out in enumerate(outs):
            assert torch.equal(out.cpu().float(), oracle.expected_combine(cfg, sources[a]).float())
        for f, rec in enumerate(received):
            exp = oracle.expected_receive(cfg, f, sources, rows=rec.recv_x.shape[0])
            assert torch.equal(rec.recv_scale.cpu()[exp.valid], exp.recv_scale[exp.valid])
    finally:
        world.close()


@pytest.mark.parametrize("kind", ["outside", "negative", "wide", "duplicate"])
def test_illegal_route_is_reported_not_trapped(kind):
    cfg = Config(16, 256, 8, 2, 2, 2, expert_alignment=4)
    world = make_world(cfg)
    try:
        batches = [list(synthetic.exact_batch(cfg, 16, a, 1)) for a in range(2)]
        ids = batches[0][1]
        if kind == "duplicate":
            ids[3, 1] = ids[3, 0]
        else:
            ids[3, 0] = {"outside": cfg.num_experts, "negative": -2, "wide": 1 << 32}[kind]
        dev = [to_dev(b) for b in batches]

        def expert(i, rec):
            return oracle.synthetic_expert_rows(cfg, i, rec.recv_x, rec.recv_scale, rec.recv_topk_weights, rec.recv_count_psum)

        outs, _ = world.exchange(dev, expert)
        torch.cuda.synchronize()
        # The offending token collects as zeros, every other token is untouched.
        expect = oracle.expected_combine(cfg, oracle.SourceBatch(*batches[0]))
        assert torch.equal(outs[0].cpu().float(), expect.float())
        assert not outs[0][3].any()
        with pytest.raises(AfdepRouteError, match="illegal route"):
            world.attention[0].check()
        world.attention[0].check()    # reported once, then cleared
        # the context is alive and the next exchange is clean
        clean = [synthetic.exact_batch(cfg, 16, a, 2) for a in range(2)]
        run_and_check(world, cfg, clean)
    finally:
        world.close()


def test_bounded_wait_reports_timeout_instead_of_hanging():
    """An FFN rank that receives without any dispatch gives up after its budget."""
    from afdep_b200 import AfdepTimeoutError

    cfg = Config(8, 256, 8, 2, 1, 1, expert_alignment=1)
    world = make_world(cfg)
    world.close()
    from afdep_b200.parallel.loopback import LoopbackWorld

    world = LoopbackWorld(cfg, gpu_timeout_s=0.05)
    try:
        rec = world.ffn[0].worker_receive(bucket=8)
        torch.cuda.synchronize()          # returns: the wait is bounded
        with pytest.raises(AfdepTimeoutError, match="counts"):
            world.ffn[0].check()
        assert rec.recv_x.shape[0] == cfg.receive_rows(8)
        # the CUDA context still works
        assert float(torch.ones(4, device="cuda").sum()) == 4.0
    finally:
        for b in world.buffers:
            b.transport._pending = None
        world.close()


def test_cuda_graph_replay_with_changed_inputs():
    cfg = Config(16, 512, 8, 2, 2, 2, expert_alignment=4)
    world = make_world(cfg)
    try:
        n, steps = 16, 3
        first = [to_dev(synthetic.exact_batch(cfg, n, a, 0)) for a in range(2)]
        static = [[t.clone() if t is not None else None for t in b] for b in first]

        def expert(i, rec):
            return oracle.synthetic_expert_rows(cfg, i, rec.recv_x, rec.recv_scale, rec.recv_topk_weights, rec.recv_count_psum)

        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(2):
                world.exchange(static, expert)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            captured = [world.exchange(static, expert)[0] for _ in range(steps)]
        for epoch in range(1, 5):
            routing = "skip" if epoch == 3 else "mixed"
            new = [synthetic.exact_batch(cfg, n, a, epoch, active=n - 3 * a, routing=routing) for a in range(2)]
            for s, b in zip(static, new):
                for dst, src in zip(s, b):
                    if dst is not None:
                        dst.copy_(src)
            graph.replay()
            torch.cuda.synchronize()
            for a in range(2):
                expect = oracle.expected_combine(cfg, oracle.SourceBatch(*new[a])).float()
                for outs in captured:
                    assert torch.equal(outs[a].cpu().float(), expect)
        for b in world.buffers:
            b.check()
    finally:
        world.close()


def _negate_(x):
    """Flip the sign of every element in place (BF16, or e4m3 through its sign bit)."""
    if x.dtype == torch.bfloat16:
        x.neg_()
    else:
        x.view(torch.uint8).bitwise_xor_(0x80)


@pytest.mark.parametrize("payload", ["bf16", "fp8"])
def test_deep_graph_of_alternating_sign_exchanges(payload):
    """24 complete exchanges per graph, the input's sign flipped in place before each one, so two
    consecutive exchanges never carry the same payload; 14 replays with routes, token counts and
    values changed in place between them (the depth of the reference's own graph check,
    tests/gpu/deepep.py:205-238).  Between replays every payload region of the heap and the
    tensors of the previous replay are overwritten with NaN bit patterns: a row read from a stale
    slot would surface as NaN."""
    cfg = Config(16, 512, 8, 2, 2, 2, expert_alignment=4, payload=payload)
    world = make_world(cfg)
    try:
        n, steps, replays = 16, 24, 14
        first = [to_dev(synthetic.exact_batch(cfg, n, a, 0)) for a in range(2)]
        static = [[t.clone() if t is not None else None for t in b] for b in first]
        leftovers = []

        def expert(i, rec):
            rows = oracle.synthetic_expert_rows(cfg, i, rec.recv_x, rec.recv_scale, rec.recv_topk_weights, rec.recv_count_psum)
            leftovers.append(rec.recv_x)
            return rows

        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(2):
                world.exchange(static, expert)
        torch.cuda.synchronize()
        leftovers.clear()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            captured = []
            for _ in range(steps):
                for b in static:
                    _negate_(b[0])
                captured.append(world.exchange(static, expert)[0])
        torch.cuda.synchronize()
        routings = ["mixed", "mixed", "skew", "skip", "mixed"]
        for epoch in range(1, replays + 1):
            routing = routings[epoch % len(routings)]
            new = [synthetic.exact_batch(cfg, n, a, epoch, active=n - (epoch + 3 * a) % 5, routing=routing) for a in range(2)]
            for s, b in zip(static, new):
                for dst, src in zip(s, b):
                    if dst is not None:
                        dst.copy_(src)
            for buf in world.buffers:
                buf._t._nb.poison_payload()
            for t in leftovers:                      # receive tensors of the captured exchanges (graph-private memory)
                t.view(torch.uint8).fill_(0xFF)
            for outs in captured:
                for o in outs:
                    o.view(torch.int16).fill_(-1)    # 0xFFFF: NaN in BF16
            graph.replay()
            torch.cuda.synchronize()
            for a in range(2):
                expect = oracle.expected_combine(cfg, oracle.SourceBatch(*new[a])).float()
                for i, outs in enumerate(captured):
                    sign = -1.0 if i % 2 == 0 else 1.0      # the i-th exchange sees the input negated i + 1 times
                    got = outs[a].cpu().float()
                    assert not torch.isnan(got).any(), f"replay {epoch}, exchange {i}: stale data"
                    assert torch.equal(got, sign * expect), f"replay {epoch}, exchange {i}, attention rank {a}"
        for b in world.buffers:
            b.check()
        assert world.buffers[0].stats()["launches"] > 0
    finally:
        world.close()


def test_eager_exchanges_survive_nan_poison_between_them():
    """Eager mode: heap payload regions and the previous exchange's receive and reply tensors are
    filled with NaN bit patterns before every exchange; results must still equal the oracle."""
    cfg = Config(64, 1024, 16, 4, 2, 2, expert_alignment=8, payload="fp8")
    world = make_world(cfg)
    try:
        stale = []
        for epoch in range(4):
            for buf in world.buffers:
                buf._t._nb.poison_payload()
            for t in stale:
                t.view(torch.uint8).fill_(0xFF)
            batches = [synthetic.exact_batch(cfg, 64 - 5 * epoch, a, epoch) for a in range(2)]
            outs, received = run_and_check(world, cfg, batches)
            stale = [r.recv_x for r in received] + [r.recv_topk_weights for r in received] + list(outs)
    finally:
        world.close()


def test_dispatch_grid_is_co_resident_or_refused():
    """The distributed-layout dispatch is a cooperative launch: with a compute kernel hogging the
    SMs on another stream it still completes (it starts once the whole grid fits), and a grid the
    GPU can never hold at once is refused on the host with an error, not left to time out."""
    cfg = Config(4096, 1024, 16, 4, 1, 1, expert_alignment=8)     # enough tokens for more CTAs than the GPU has SMs
    world = make_world(cfg)
    try:
        batches = [synthetic.random_batch(cfg, 4096, seed=3)]
        side = torch.cuda.Stream()
        a = torch.randn(8192, 8192, device="cuda", dtype=torch.bfloat16)
        with torch.cuda.stream(side):
            for _ in range(6):
                a @ a                                 # a few milliseconds of GEMMs that fill every SM
        run_and_check(world, cfg, batches, exact=False)
        side.synchronize()
        sms = torch.cuda.get_device_properties(0).multi_processor_count
        att = world.attention[0]
        att._t._nb.set_dispatch_ctas(min(160, sms + 12))
        if sms + 12 <= 160:
            x, ids, w, _ = to_dev(batches[0])
            with pytest.raises(RuntimeError, match="dispatch launch"):
                att.source_dispatch(x, ids, w, None, bucket=4096)
            att.transport._pending = None
            torch.cuda.synchronize()
            att._t._nb.set_dispatch_ctas(sms)
            run_and_check(world, cfg, batches, exact=False)      # the Buffer is still usable
    finally:
        world.close()


def test_int32_expert_ids():
    """The 32-bit index build of the reference (EP_NUM_TOPK_IDX_BITS=32) as a Buffer option."""
    cfg = Config(48, 512, 16, 4, 2, 2, expert_alignment=8)
    world = make_world(cfg, topk_idx_bits=32)
    try:
        assert world.attention[0].topk_idx_dtype == torch.int32
        batches = [synthetic.exact_batch(cfg, 48 - 5 * a, a, 1) for a in range(2)]
        dev = [(x.cuda(), ids.to(torch.int32).cuda(), w.cuda(), None) for x, ids, w, _ in batches]

        def expert(i, rec):
            return oracle.synthetic_expert_rows(cfg, i, rec.recv_x, rec.recv_scale, rec.recv_topk_weights, rec.recv_count_psum)

        outs, _ = world.exchange(dev, expert)
        torch.cuda.synchronize()
        for a, out in enumerate(outs):
            assert torch.equal(out.cpu().float(), oracle.expected_combine(cfg, oracle.SourceBatch(*batches[a])).float())
        with pytest.raises(ValueError):
            world.attention[0].source_dispatch(dev[0][0], batches[0][1].cuda(), dev[0][2], None, bucket=48)     # int64 ids into a 32-bit Buffer
        for b in world.buffers:
            b.check()
    finally:
        world.close()


def test_async_finish_hands_back_an_event():
    """Role calls on the dedicated communication stream that do not make the caller's stream wait:
    the caller joins through the EventHandle (the reference's async / EventHandle mode,
    csrc/utils/event.hpp:10-42)."""
    cfg = Config(32, 512, 8, 2, 1, 1, expert_alignment=8)
    world = make_world(cfg, use_comm_stream=True)
    try:
        att, ffn = world.attention[0], world.ffn[0]
        batch = synthetic.exact_batch(cfg, 32, 0, 2)
        x, ids, w, _ = to_dev(batch)
        handle = att.source_dispatch(x, ids, w, None, bucket=32, async_finish=True)
        assert handle is not None and hasattr(handle, "current_stream_wait")
        handle.current_stream_wait()
        rec = ffn.worker_receive(bucket=32)
        rows = oracle.synthetic_expert_rows(cfg, 0, rec.recv_x, rec.recv_scale, rec.recv_topk_weights, rec.recv_count_psum)
        done = ffn.worker_reply(rows, rec.receipt, async_finish=True)
        done.current_stream_wait()
        out = att.source_collect()
        torch.cuda.synchronize()
        assert done.query()
        assert torch.equal(out.cpu().float(), oracle.expected_combine(cfg, oracle.SourceBatch(*batch)).float())
        for b in world.buffers:
            b.check()
    finally:
        world.close()


def test_dedicated_comm_stream_option():
    """Exchange kernels on a separate high-priority stream, ordered with events."""
    cfg = Config(32, 512, 8, 2, 2, 2, expert_alignment=8)
    world = make_world(cfg, use_comm_stream=True)
    try:
        assert world.buffers[0].comm_stream != torch.cuda.current_stream()
        for epoch in range(2):
            batches = [synthetic.exact_batch(cfg, 32, a, epoch) for a in range(2)]
            run_and_check(world, cfg, batches)
    finally:
        world.close()


def test_expert_stats_accumulate_on_the_device():
    """Optional running totals of rows received per local expert, eager and host-count paths."""
    cfg = Config(64, 256, 16, 4, 2, 2, expert_alignment=8)
    world = make_world(cfg, expert_stats=True)
    try:
        want = torch.zeros(cfg.num_experts, dtype=torch.int64)
        for epoch, host in enumerate((False, True, False)):
            batches = [synthetic.random_batch(cfg, 64 - 9 * a, seed=5 * epoch + a, skip_fraction=0.1) for a in range(2)]
            run_and_check(world, cfg, batches, read_host_counts=host, exact=False)
            for b in batches:
                ids = b[1][b[1] >= 0]
                want += torch.bincount(ids, minlength=cfg.num_experts)
        el = cfg.experts_per_rank
        for f in range(cfg.ffn_ranks):
            got = world.buffers[f].stats()["expert_rows_received"]
            assert got == want[f * el : (f + 1) * el].tolist()
        assert "expert_rows_received" not in world.buffers[cfg.ffn_ranks].stats()      # attention rank
    finally:
        world.close()


@pytest.mark.parametrize("hidden,ffn,attn", [(1024, 2, 2), (768, 1, 3), (7168, 2, 2)])
def test_scales_as_packed_exponent_bytes(hidden, ffn, attn):
    """``scale_format="ue8m0x4"``: the FP8 rows' scales travel as int32 words of four exponent bytes
    (6 scales pad to 2 words at hidden 768) and come back bit for bit, in the column-major layout too."""
    cfg = Config(64, hidden, 16, 4, ffn, attn, expert_alignment=8, payload="fp8", scale_format="ue8m0x4")
    assert cfg.scale_groups == (hidden // 128 + 3) // 4
    world = make_world(cfg)
    try:
        for epoch in range(2):
            batches = [synthetic.exact_batch(cfg, 64 - 9 * a, a, epoch) for a in range(attn)]
            assert all(b[3].dtype == torch.int32 and b[3].shape[1] == cfg.scale_groups for b in batches)
            _, received = run_and_check(world, cfg, batches)
            assert all(r.recv_scale.dtype == torch.int32 and r.recv_scale.stride(0) == 1 for r in received)
        batches = [synthetic.random_batch(cfg, 50, 3 + a, zipf_s=1.1) for a in range(attn)]
        run_and_check(world, cfg, batches)
        x, ids, w, scale = to_dev(batches[0])
        with pytest.raises(ValueError, match="dtype, shape"):
            world.attention[0].source_dispatch(x, ids, w, torch.ones((x.shape[0], hidden // 128), device="cuda"), bucket=64)
    finally:
        world.close()
