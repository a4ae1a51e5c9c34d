"""All-gather, send/recv and row fetch on the heap's auxiliary region (one GPU, loopback world).

In a loopback world the ranks' kernels run one after another on one stream, so every push is
issued before the matching wait, exactly as the module docstring of the loopback world asks.
"""

import pytest
import torch

from afdep_b200 import Config
from afdep_b200.parallel.primitives import HeapPrimitives

pytestmark = pytest.mark.gpu


@pytest.fixture
def world():
    from afdep_b200.parallel.loopback import LoopbackWorld

    cfg = Config(8, 256, 8, 2, 2, 2)
    w = LoopbackWorld(cfg, gpu_timeout_s=2.0, aux_bytes=8 << 20)
    yield w
    w.close()


def test_all_gather(world):
    prims = [HeapPrimitives(b) for b in world.buffers]
    for rnd in range(3):
        parts = [torch.full((33, 64), float(10 * rnd + r), device="cuda", dtype=torch.bfloat16) + torch.arange(64, device="cuda") for r in range(4)]
        handles = [p.all_gather_start(t) for p, t in zip(prims, parts)]
        for h in handles:
            got = h.wait()
            torch.cuda.synchronize()
            assert torch.equal(got, torch.stack(parts))
    for b in world.buffers:
        b.check()


def test_all_gather_copy_engine_and_mixed(world):
    """Copy-engine pushes with stream-ordered flag writes; ranks may mix the two engines, and
    the two forms may alternate from one gather to the next."""
    prims = [HeapPrimitives(b) for b in world.buffers]
    for rnd, engines in enumerate((["copy"] * 4, ["copy", "sm", "copy", "sm"], ["sm"] * 4, ["copy"] * 4)):
        parts = [torch.randn(40, 64, device="cuda").bfloat16() + rnd for _ in range(4)]
        handles = [p.all_gather_start(t, engine=e) for p, t, e in zip(prims, parts, engines)]
        for h in handles:
            got = h.wait()
            torch.cuda.synchronize()
            assert torch.equal(got, torch.stack(parts))
    with pytest.raises(ValueError):
        prims[0].all_gather_start(parts[0], engine="dma")
    for b in world.buffers:
        b.check()


def test_send_recv_ring_with_credits(world):
    """Four messages per pair in flight before the first receive (the ring's depth), twice over,
    so the second batch of sends runs on credits returned by the first batch of receives."""
    prims = [HeapPrimitives(b) for b in world.buffers]
    n = len(prims)
    depth = prims[0].inflight
    assert depth == 4
    for batch in range(2):
        msgs = [[torch.randn(3000, device="cuda") + 10 * r + k for k in range(depth)] for r in range(n)]
        for k in range(depth):
            for r, p in enumerate(prims):
                p.send(msgs[r][k], (r + 1) % n)
        for k in range(depth):
            for r, p in enumerate(prims):
                out = torch.empty(3000, device="cuda")
                p.recv(out, (r - 1) % n)
                torch.cuda.synchronize()
                assert torch.equal(out, msgs[(r - 1) % n][k]), (batch, k, r)
    for b in world.buffers:
        b.check()


def test_large_message_through_the_copy_pipeline(world):
    """A message of many 32 KB chunks over several CTAs, with a ragged tail."""
    prims = [HeapPrimitives(b) for b in world.buffers]
    nbytes = min(prims[0].message_bytes, (200 << 10) + 48)
    src = torch.randint(0, 255, (nbytes,), device="cuda", dtype=torch.uint8)
    out = torch.zeros_like(src)
    prims[0].send(src, 2)
    prims[2].recv(out, 0)
    torch.cuda.synchronize()
    assert torch.equal(out, src)
    world.buffers[0].check()


def test_back_to_back_gathers_without_barrier(world):
    prims = [HeapPrimitives(b) for b in world.buffers]
    results, inputs = [], []
    for rnd in range(5):
        parts = [torch.randn(24, 64, device="cuda").bfloat16() + rnd for _ in range(4)]
        inputs.append(torch.stack(parts))
        handles = [p.all_gather_start(t) for p, t in zip(prims, parts)]
        results.append([h.wait() for h in handles])
    torch.cuda.synchronize()
    for want, got in zip(inputs, results):
        for g in got:
            assert torch.equal(g, want)


def test_fetch_rows(world):
    prims = [HeapPrimitives(b) for b in world.buffers]
    rows, width = 50, 128
    table = torch.randn(4 * rows, width, device="cuda").bfloat16()
    for r, p in enumerate(prims):
        p.table_shard(rows, width, torch.bfloat16).copy_(table[r * rows : (r + 1) * rows])
    torch.cuda.synchronize()
    idx = torch.randint(0, 4 * rows, (300,), device="cuda")
    idx[0] = -5                      # out of range: a zero row, not a wild read
    want = table[idx.clamp(min=0)]
    want[0] = 0
    for p in prims:
        got = p.fetch_rows(idx, rows, width, torch.bfloat16)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    # issue / wait split: the fetch runs on a side stream while this stream does other work
    handle = prims[1].fetch_rows_start(idx, rows, width, torch.bfloat16)
    other = torch.randn(256, 256, device="cuda") @ torch.randn(256, 256, device="cuda")
    got = handle.wait()
    torch.cuda.synchronize()
    assert torch.equal(got, want) and bool(torch.isfinite(other).all())
    # rows wider than the per-warp bulk buffer take the plain-load path
    wide = prims[0].table_shard(2, 8192, torch.bfloat16)
    wide.copy_(torch.arange(2 * 8192, device="cuda").view(2, 8192).bfloat16())
    torch.cuda.synchronize()
    got = prims[3].fetch_rows(torch.tensor([1, 0], device="cuda"), 2, 8192, torch.bfloat16)
    torch.cuda.synchronize()
    assert torch.equal(got, wide[[1, 0]])
