"""NVLink rate between two GPUs as this library's own copy kernels reach it.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 \
        bench_nvlink.py [--mb 64] [--iters 20] [--inflight 4]

Two ranks of one Buffer exchange messages through the heap's neighbour send/recv primitive
(bulk asynchronous copies staged through shared memory, `csrc/kernels/aux.cu`): one message,
a stream of messages one way, then streams both ways at once, timed on the device with CUDA
events on each side.  The send kernel ends when its stores have been performed at the peer, so
its time alone is the link rate a copy kernel of this library reaches (the denominator `bench.py`
quotes as "measured rate" next to the nominal 900 GB/s per direction); "delivered" figures end
when the receiver has copied the message out of its heap.
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
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--messages", type=int, default=16, help="messages per timed stream")
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

    def stream_of(count: int, send: bool, recv: bool) -> float:
        """Device time for `count` messages in a row (sender and receiver each issue all of theirs)."""
        prim.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if send and recv:           # both directions: sends and receives interleaved so that credits keep flowing
            for _ in range(count):
                prim.send(src, peer)
                prim.recv(dst, peer)
        elif send:
            for _ in range(count):
                prim.send(src, peer)
        elif recv:
            for _ in range(count):
                prim.recv(dst, peer)
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1)

    def best(count, send, recv):
        stream_of(min(count, a.inflight), send, recv)            # warm-up
        return min(stream_of(count, send, recv) for _ in range(a.iters))

    single = best(1, rank == 0, rank == 1)                        # one message: the send, then its copy-out
    one_way = best(a.messages, rank == 0, rank == 1)              # a stream of messages: copy-outs overlap later sends
    both = best(a.messages, True, True)
    torch.cuda.synchronize()
    ok = bool((dst == peer + 1).all())
    buf.check()
    gathered = [None, None]
    dist.all_gather_object(gathered, (single, one_way, both, ok))
    if rank == 0:
        gbs = lambda ms, n: round(n * nbytes / (ms * 1e-3) / 1e9, 1)      # noqa: E731
        print(json.dumps({
            "probe": "neighbour send/recv over the symmetric heap, 2 GPUs",
            "message_mib": a.mb,
            "messages_per_stream": a.messages,
            "inflight_slots": a.inflight,
            "send_kernel_alone_GBs": gbs(gathered[0][0], 1),
            "single_message_delivered_GBs": gbs(gathered[1][0], 1),
            "stream_sender_side_GBs": gbs(gathered[0][1], a.messages),
            "stream_delivered_GBs": gbs(gathered[1][1], a.messages),
            "both_ways_delivered_GBs_per_direction": gbs(max(g[2] for g in gathered), a.messages),
            "payload_verified": all(g[3] for g in gathered),
            "timing": "CUDA events around the kernels of each side, best of %d after warm-up; 'send kernel alone' ends when its "
                      "stores have been performed at the peer, 'delivered' when the receiver has copied the message out of its heap" % a.iters,
        }))
    buf.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
