"""Run a function as N ranks of a CPU Gloo job (child processes, rendezvous on 127.0.0.1)."""

from __future__ import annotations

import os
import socket
import traceback

import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, errors):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    try:
        import datetime

        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))
        fn(rank, world, *args)
        dist.barrier()
        dist.destroy_process_group()
    except BaseException:  # noqa: BLE001
        errors.put((rank, traceback.format_exc()))
        raise


def run_ranks(fn, world: int, *args, timeout: float = 300.0) -> None:
    ctx = mp.get_context("spawn")
    errors = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, errors)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.kill()
    msgs = []
    while not errors.empty():
        msgs.append("rank %d:\n%s" % errors.get())
    assert not alive, "ranks timed out"
    assert not msgs and all(p.exitcode == 0 for p in procs), "\n".join(msgs) or [p.exitcode for p in procs]
