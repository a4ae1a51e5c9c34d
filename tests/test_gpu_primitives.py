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
    w = LoopbackWorld(cfg, gpu_timeout_s=2.0, aux_bytes=4 << 20)
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
    prims = [HeapPrimitives(b) for b in world.buffers]
    n = len(prims)
    for step in range(4):      # more messages than slots: every send needs the previous credit
        msgs = [torch.randn(1024, device="cuda") + r for r in range(n)]
        for r, p in enumerate(prims):
            p.send(msgs[r], (r + 1) % n)
        for r, p in enumerate(prims):
            out = torch.empty(1024, device="cuda")
            p.recv(out, (r - 1) % n)
            torch.cuda.synchronize()
            assert torch.equal(out, msgs[(r - 1) % n])
    for b in world.buffers:
        b.check()


def test_fetch_rows(world):
    prims = [HeapPrimitives(b) for b in world.buffers]
    rows, width = 50, 128
    table = torch.randn(4 * rows, width, device="cuda").bfloat16()
    for r, p in enumerate(prims):
        p.table_shard(rows, width, torch.bfloat16).copy_(table[r * rows : (r + 1) * rows])
    torch.cuda.synchronize()
    idx = torch.randint(0, 4 * rows, (300,), device="cuda")
    idx[0] = -5                      # out of range: a zero row, not a wild read
    for p in prims:
        got = p.fetch_rows(idx, rows, width, torch.bfloat16)
        torch.cuda.synchronize()
        want = table[idx.clamp(min=0)]
        want[0] = 0
        assert torch.equal(got, want)
