"""Timed CPU baseline: the exchange on the pure-torch Gloo transport (no GPU involved).

    python bench_cpu_oracle.py [--steps 20]

Four CPU ranks (0-1 FFN, 2-3 attention), hidden 256 (the API needs a multiple of 256; the
benchmark description names 128), 8 experts, top-2, 16 tokens per attention rank, bucket 16.
The synthetic expert returns row * (e + 1), weighted by the caller; every step checks
out == sum_k w_k (e_k + 1) x and the reported time is the maximum over ranks of the mean
wall-clock per exchange.
"""

from __future__ import annotations

import argparse
import json
import os
import socket
import time

import torch
import torch.multiprocessing as mp


def _rank(rank: int, world: int, port: int, steps: int, out) -> None:
    import torch.distributed as dist

    from afdep_b200 import Buffer, Config
    from afdep_b200.utils import oracle, synthetic

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = Config(16, 256, 8, 2, 2, 2, expert_alignment=16)
    buf = Buffer(group=dist.group.WORLD, config=cfg, backend="gloo")
    times = []
    for step in range(steps + 3):
        batches = [synthetic.random_batch(cfg, 16, seed=31 * step + a) for a in range(2)]
        dist.barrier()
        t0 = time.perf_counter()
        if buf.role == "attention":
            x, ids, w, _ = batches[buf.role_rank]
            buf.source_dispatch(x, ids, w, bucket=16)
            got = buf.source_collect()
        else:
            rec = buf.worker_receive(bucket=16)
            rows = oracle.synthetic_expert_rows(cfg, buf.role_rank, rec.recv_x, None, rec.recv_topk_weights, rec.recv_count_psum)
            buf.worker_reply(rows, rec.receipt)
        dt = time.perf_counter() - t0
        if step >= 3:
            times.append(dt)
        if buf.role == "attention":
            want = oracle.expected_combine(cfg, oracle.SourceBatch(x, ids, w))
            assert torch.equal(got.float(), want.float())
    mean = torch.tensor([sum(times) / len(times)])
    dist.all_reduce(mean, op=dist.ReduceOp.MAX)
    buf.close()
    if rank == 0:
        out.put(float(mean))
    dist.destroy_process_group()


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--steps", type=int, default=20)
    a = p.parse_args()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 4, port, a.steps, out)) for r in range(4)]
    for q in procs:
        q.start()
    for q in procs:
        q.join()
    print(json.dumps({"impl": "gloo-cpu", "ranks": 4, "config": "hidden 256, 8 experts, top-2, 16 tokens/rank", "steps": a.steps,
                      "ms_per_exchange": round(out.get() * 1e3, 3), "checked": "out == sum_k w_k (e_k+1) x, bit-exact"}))


if __name__ == "__main__":
    main()
