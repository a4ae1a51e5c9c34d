"""NVLink rate between two GPUs as this library's own copy kernels reach it.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 \
        bench_nvlink.py [--mb 64] [--iters 20] [--inflight 4]

Two ranks of one Buffer exchange messages through the heap's neighbour send/recv primitive
(bulk asynchronous copies staged through shared memory, `csrc/kernels/aux.cu`): first one way,
then both ways at once.  Each message is timed on the device with CUDA events on both sides
(the later of "send kernel done" and "receive kernel done"), after warm-up, the maximum over the
two ranks is taken, and rank 0 prints one JSON line.  The one-way figure is the denominator
`bench.py` quotes as "measured rate" next to the nominal 900 GB/s per direction.
"""

from __future__ import annotations

import argparse
import datetime
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--mb", type=int, default=64, help="message size in MiB")
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--inflight", type=int, default=4, help="messages a sender may have in flight")
    a = p.parse_args()

    import torch
    import torch.distributed as dist

    from afdep_b200 import Buffer, Config
    from afdep_b200.parallel.primitives import HeapPrimitives

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    assert world == 2, "run on exactly two GPUs"
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=300))
    nbytes = a.mb << 20
    cfg = Config(16, 256, 2, 1, 1, 1, gpu_timeout_s=20)
    buf = Buffer(group=dist.group.WORLD, config=cfg, aux_bytes=world * a.inflight * nbytes + (1 << 20), p2p_inflight=a.inflight)
    prim = HeapPrimitives(buf)
    peer = 1 - rank
    src = torch.full((nbytes,), rank + 1, dtype=torch.uint8, device="cuda")
    dst = torch.empty_like(src)

    def timed(send: bool, recv: bool) -> float:
        times = []
        for i in range(3 + a.iters):
            prim.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if send:
                prim.send(src, peer)
            if recv:
                prim.recv(dst, peer)
            e1.record()
            e1.synchronize()
            if i >= 3:
                times.append(e0.elapsed_time(e1))
        return sum(times) / len(times)

    one_way = timed(send=rank == 0, recv=rank == 1)
    both = timed(send=True, recv=True)
    torch.cuda.synchronize()
    ok = bool((dst == peer + 1).all())
    buf.check()
    gathered = [None, None]
    dist.all_gather_object(gathered, (one_way, both, ok))
    if rank == 0:
        ms_one = max(g[0] for g in gathered)
        ms_both = max(g[1] for g in gathered)
        print(json.dumps({
            "probe": "neighbour send/recv over the symmetric heap, 2 GPUs",
            "message_mib": a.mb,
            "inflight_slots": a.inflight,
            "one_way_GBs": round(nbytes / (ms_one * 1e-3) / 1e9, 1),
            "both_ways_GBs_per_direction": round(nbytes / (ms_both * 1e-3) / 1e9, 1),
            "ms_one_way": round(ms_one, 4),
            "ms_both_ways": round(ms_both, 4),
            "payload_verified": all(g[2] for g in gathered),
            "timing": "CUDA events around send and receive kernels, mean of %d after 3 warm-ups, max over the two ranks" % a.iters,
        }))
    buf.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
