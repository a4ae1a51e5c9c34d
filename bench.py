"""Headline benchmark: dispatch + combine of one AFD expert-parallel exchange.

    python bench.py --gpus N --steps K --warmup W [--impl ours|nccl|reference] [--config weak|2|3|4]

N = 1 runs one attention and one FFN rank colocated on a single GPU (all ranks in this
process); N >= 2 expects one process per GPU (torchrun) and splits the ranks N/2 FFN + N/2
attention (6 attention + 2 FFN for ``--config 4``).  A step is one complete exchange through
the public role API: ``source_dispatch`` -> ``worker_receive`` -> ``worker_reply`` ->
``source_collect``.  The FFN "expert" is the identity on a preallocated BF16 tensor, so the
timed region holds the library's four kernels and nothing else.

Every step is bracketed by CUDA events on the launching stream after a device-side barrier
across ranks (outside the events); L2 is flushed between steps; the reported time is the
maximum over ranks.  ``value`` is the job's aggregate wire throughput: bytes that cross NVLink
in both directions (one record per token and destination FFN rank out, one BF16 row back)
divided by the step time.  The ``e2e`` entry repeats the measurement with, inside the timed
region, the host->device copy of the step's inputs from pinned memory and a device->host read
of a checksum of the result.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # name: hidden, experts per FFN rank, top_k, tokens per attention rank, payload, routing
    "weak": dict(hidden=4096, experts_per_ffn=64, top_k=8, tokens=2048, payload="bf16", zipf=None),
    "2": dict(hidden=4096, experts_per_ffn=64, top_k=8, tokens=2048, payload="bf16", zipf=None),
    "3": dict(hidden=7168, experts_per_ffn=64, top_k=8, tokens=4096, payload="fp8", zipf=1.1),
    "4": dict(hidden=7168, experts_per_ffn=128, top_k=8, tokens=128, payload="bf16", zipf=None),
    # end-to-end MoE layer: the FFN ranks run SwiGLU experts 7168 -> 2048 -> 7168 on tcgen05
    "5": dict(hidden=7168, experts_per_ffn=64, top_k=8, tokens=2048, payload="fp8", zipf=None, intermediate=2048),
}


def parse_args():
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=50)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", choices=("ours", "nccl", "reference"), default="ours")
    p.add_argument("--config", choices=tuple(CONFIGS), default="weak")
    p.add_argument("--expert-weights", choices=("fp8", "bf16"), default="fp8", help="config 5: storage of the expert weights")
    p.add_argument("--expert-down", choices=("fp8", "bf16"), default=None, help="config 5: storage of the down projection (default: like --expert-weights)")
    p.add_argument("--tokens", type=int, default=0, help="override tokens per attention rank")
    p.add_argument("--num-sms", type=int, default=0)
    p.add_argument("--graph", action="store_true", help="(default for --impl ours) replay each timed step from a CUDA graph")
    p.add_argument("--eager", action="store_true", help="time eager launches instead of CUDA-graph replays")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--trace", action="store_true", help="print per-kernel device time stamps of the last step (native transport)")
    return p.parse_args()


def topology(n: int, config: str) -> tuple[int, int]:
    if n == 1:
        return 1, 1
    if config == "4" and n == 8:
        return 2, 6
    return n // 2, n - n // 2


class ClockSampler:
    """SM clock and throttle reasons while the timed region runs.  Read-only NVML queries from
    a background thread (about every millisecond); falls back to one `nvidia-smi` query if NVML is missing."""

    REASONS = {
        "hw_slowdown": 0x8,
        "sw_power_cap": 0x4,
        "sw_thermal_slowdown": 0x20,
        "hw_thermal_slowdown": 0x40,
    }

    def __init__(self, device_index: int) -> None:
        self.index, self.samples, self.reasons, self.max_mhz = device_index, [], set(), None
        self._stop, self._thread, self._nvml = False, None, None

    def _loop(self) -> None:
        nv, h = self._nvml, self._handle
        while not self._stop:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for name, bit in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001 - sampling must never break the benchmark
                pass
            time.sleep(0.0005)

    def start(self) -> None:
        try:
            import pynvml as nv

            nv.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = int(visible.split(",")[self.index]) if visible and visible.split(",")[self.index].isdigit() else self.index
            self._handle = nv.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(self._handle, nv.NVML_CLOCK_SM)
            self._nvml = nv
            import threading

            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        except Exception:  # noqa: BLE001
            self._nvml = None

    def stop(self) -> dict:
        if self._nvml is not None:
            self._stop = True
            self._thread.join(timeout=1.0)
            return {
                "sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz,
                "samples": len(self.samples),
                "reasons": sorted(self.reasons),
                "source": "nvml",
            }
        try:
            out = subprocess.run(
                ["nvidia-smi", "--query-gpu=clocks.sm,clocks.max.sm", "--format=csv,noheader,nounits", "-i", str(self.index)],
                capture_output=True, text=True, timeout=10,
            ).stdout.strip().split(",")
            return {"sm_mhz": float(out[0]), "sm_max_mhz": float(out[1]), "samples": 1, "reasons": [], "source": "nvidia-smi after the run"}
        except Exception:  # noqa: BLE001
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["clock query unavailable"]}


def reference_arm(args) -> None:
    """The unmodified reference cannot run on this pool; say why in one line."""
    rank = int(os.environ.get("RANK", "0"))
    reason = None
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "afdep")):
        reason = (
            "closed on this pool: the reference's source calls a batched-memcpy CUDA entry point that is closed here "
            "(csrc/elastic/buffer.hpp:439), so its install under baseline/_ref cannot be carried to the GPU box"
        )
        if args.gpus < 2:
            reason += "; it also has no 1-GPU mode (needs at least two ranks, afdep/deepep.py:218-221)"
    elif args.gpus < 2:
        reason = "the reference needs at least two ranks (afdep/deepep.py:218-221); there is no 1-GPU mode"
    else:
        probe = (
            "import sys; sys.path.insert(0, %r); from afdep._build import load_deepep; load_deepep(); print('built')" % ref
        )
        try:
            out = subprocess.run([sys.executable, "-c", probe], capture_output=True, text=True, timeout=900)
            if out.returncode != 0:
                tail = (out.stderr.strip().splitlines() or ["build failed"])[-1]
                reason = "reference extension does not build here (needs NCCL >= 2.30.7 device API): " + tail[:200]
            else:
                reason = "reference built, but its run-time JIT shells out to cuobjdump for every kernel, which is not allowed here"
        except subprocess.TimeoutExpired:
            reason = "reference extension build timed out"
    if rank == 0:
        print(json.dumps({"impl": "reference", "unavailable": reason}))


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    from afdep_b200 import Buffer, Config
    from afdep_b200.utils import synthetic

    n = args.gpus
    spec = dict(CONFIGS[args.config])
    if args.tokens:
        spec["tokens"] = args.tokens
    ffn, attn = topology(n, args.config)
    T = spec["tokens"]
    cfg = Config(
        T,
        spec["hidden"],
        spec["experts_per_ffn"] * ffn,
        spec["top_k"],
        ffn,
        attn,
        payload=spec["payload"],
        num_sms=args.num_sms,
        gpu_timeout_s=20,
        cpu_timeout_s=60,
    )
    multi = n > 1
    if multi:
        rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        assert world == n, "launch with torchrun --nproc-per-node equal to --gpus"
        local = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(local)
        import datetime

        dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=600))
        backend = "native" if args.impl == "ours" else "nccl"
        buffers = [Buffer(group=dist.group.WORLD, config=cfg, backend=backend)]
    else:
        rank, local = 0, 0
        torch.cuda.set_device(0)
        if args.impl != "ours":
            print(json.dumps({"impl": args.impl, "unavailable": "the NCCL baseline needs at least two ranks"}))
            return
        from afdep_b200.parallel.loopback import LoopbackWorld

        world_obj = LoopbackWorld(cfg, gpu_timeout_s=20.0)
        buffers = world_obj.buffers
    dev = torch.device("cuda", local)

    # ---- per-rank state: pinned host inputs, device inputs, identity-expert rows ----------
    state = []
    for buf in buffers:
        s = {"buf": buf}
        if buf.role == "attention":
            x, ids, w, scale = synthetic.random_batch(cfg, T, seed=1000 + buf.role_rank, zipf_s=spec["zipf"])
            s["host"] = [t.pin_memory() if t is not None else None for t in (x, ids, w, scale)]
            s["dev"] = [t.to(dev) if t is not None else None for t in s["host"]]
            s["ids_cpu"] = ids
        elif "intermediate" in spec:
            from afdep_b200.models.moe_layer import ExpertWeights

            s["weights"] = ExpertWeights.random(
                cfg.experts_per_rank, cfg.hidden_size, spec["intermediate"], mode=args.expert_weights, down=args.expert_down, seed=7 + buf.role_rank, device=dev
            )
        else:
            s["rows"] = torch.zeros((cfg.receive_rows(T), cfg.hidden_size), dtype=torch.bfloat16, device=dev)
        state.append(s)

    # wire bytes per step (both directions) from the routes: one record per (token, FFN rank)
    el = cfg.experts_per_rank
    per_ffn = [0] * ffn          # records this process's attention ranks send to each FFN rank
    egress = []                  # records leaving each local attention rank
    for s in state:
        if "ids_cpu" in s:
            ids = s["ids_cpu"]
            dest = torch.where(ids >= 0, ids // el, torch.full_like(ids, -1))
            mine = [int((dest == f).any(dim=1).sum()) for f in range(ffn)]
            per_ffn = [p + m for p, m in zip(per_ffn, mine)]
            egress.append(sum(mine))
    if multi:
        gathered = [None] * n
        dist.all_gather_object(gathered, (per_ffn, egress))
        per_ffn = [sum(g[0][f] for g in gathered) for f in range(ffn)]
        egress = [e for g in gathered for e in g[1]]
    records = sum(per_ffn)
    row_out = cfg.hidden_size * (1 if cfg.is_fp8 else 2) + (cfg.scale_groups * 4 if cfg.is_fp8 else 0)
    row_back = cfg.hidden_size * 2
    wire_bytes = records * (row_out + row_back)
    # NVLink roofline: bytes through the busiest port (an attention rank's egress or an FFN
    # rank's ingress on dispatch, the reverse on combine) over the measured 770 GB/s per direction.
    busiest = max(max(egress, default=0), max(per_ffn, default=0))
    roofline = {
        "busiest_port_records": busiest,
        "dispatch_us_at_770GBs": round(busiest * row_out / 770e9 * 1e6, 2),
        "combine_us_at_770GBs": round(busiest * row_back / 770e9 * 1e6, 2),
        "dispatch_us_at_900GBs_nominal": round(busiest * row_out / 900e9 * 1e6, 2),
        "combine_us_at_900GBs_nominal": round(busiest * row_back / 900e9 * 1e6, 2),
        "note": "colocated ranks share one GPU: no NVLink, HBM-bound" if not multi else "",
    }

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ordered = sorted(state, key=lambda s: 0 if s["buf"].role == "attention" else 1)

    def barrier_all():
        if multi:
            buffers[0]._t._nb.barrier() if args.impl == "ours" else dist.barrier()

    phase_log: dict[str, list] = {"dispatch": [], "receive": [], "experts": [], "reply": [], "collect": []}

    def mark(name, fn, record):
        if not record:
            return fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        out = fn()
        b.record()
        phase_log[name].append((a, b))
        return out

    def step(copy_inputs: bool, record: bool = False):
        """One exchange in dependency order; returns the collected output on attention ranks."""
        result = None
        for s in ordered:
            if s["buf"].role == "attention":
                if copy_inputs:
                    for d, h in zip(s["dev"], s["host"]):
                        if d is not None:
                            d.copy_(h, non_blocking=True)
                x, ids, w, scale = s["dev"]
                mark("dispatch", lambda: s["buf"].source_dispatch(x, ids, w, scale, bucket=T), record)
        for s in ordered:
            if s["buf"].role == "ffn":
                rec = mark("receive", lambda: s["buf"].worker_receive(bucket=T), record)
                if "weights" in s:
                    from afdep_b200.models.moe_layer import run_experts

                    rows = mark("experts", lambda: run_experts(rec, s["weights"], cfg.expert_alignment), record)
                else:
                    rows = rec.recv_x if not cfg.is_fp8 else s["rows"]
                s["psum"] = rec.recv_count_psum
                mark("reply", lambda: s["buf"].worker_reply(rows, rec.receipt), record)
        for s in ordered:
            if s["buf"].role == "attention":
                s["out"] = mark("collect", lambda: s["buf"].source_collect(), record)
                result = s["out"]
        return result

    def count_launches():
        return sum(int(s["buf"].stats().get("launches", 0)) for s in state)

    # kernels of this library per exchange on this process, counted on one eager warm-up step
    before_one = count_launches()
    step(False)
    torch.cuda.synchronize()
    launches_per_step = count_launches() - before_one
    if multi:
        dist.barrier()

    use_graph = args.impl == "ours" and not args.eager
    graph = None
    if use_graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                step(False)
        torch.cuda.synchronize()
        if multi:
            dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            step(False)
        torch.cuda.current_stream().wait_stream(side)

    def timed(copy_inputs: bool, steps: int, warmup: int):
        """Device time of each step.  The kernel-only pass enqueues every step back to back (the
        L2 flush and the cross-rank barrier sit between the event pairs, outside them) and
        synchronises once; the end-to-end pass waits for each step's result on the host."""
        pairs = []
        host_result = torch.zeros(1, dtype=torch.float32).pin_memory()
        for i in range(warmup + steps):
            flush.fill_(i & 0xFF)
            barrier_all()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if graph is not None and not copy_inputs:
                graph.replay()
            else:
                out = step(copy_inputs, record=(i >= warmup and not copy_inputs))
                if copy_inputs:
                    src = out.float().sum().reshape(1) if out is not None else state[0]["psum"].float().sum().reshape(1)
                    host_result.copy_(src, non_blocking=True)
            e1.record()
            if copy_inputs:
                e1.synchronize()
            pairs.append((e0, e1))
        torch.cuda.synchronize()
        return [a.elapsed_time(b) for a, b in pairs[warmup:]]

    traces = []
    if args.trace and args.impl == "ours":
        traces = [(s["buf"].rank, s["buf"]._t._nb.trace(True)) for s in state]
    torch.cuda.synchronize()
    if multi:
        dist.barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    torch.cuda.synchronize()
    t_wall0 = time.perf_counter()
    times = timed(False, args.steps, args.warmup)
    torch.cuda.synchronize()
    t_wall1 = time.perf_counter()
    clocks_timed_region_samples = len(sampler.samples) if rank == 0 else 0
    launches = launches_per_step * args.steps      # every timed step replays / launches the same kernels
    if graph is not None:
        # per-call device times come from a short eager pass; the headline stays the graph replay
        saved, graph = graph, None
        timed(False, min(args.steps, 10), 2)
        graph = saved
    e2e_times = None
    if not args.no_e2e:
        e2e_times = timed(True, args.steps, max(3, args.warmup))

    # the sampler keeps running through the eager and end-to-end passes: all of it is under load
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["samples_in_device_timed_region"] = clocks_timed_region_samples

    def reduce_max(values):
        total = sum(values)
        if multi:
            allv = [None] * n
            dist.all_gather_object(allv, total)
            return max(allv)
        return total

    # mean device time of each role call (kernel plus its waits), maximum over ranks
    phases = {}
    for name, pairs in phase_log.items():
        local_us = 1e3 * sum(a.elapsed_time(b) for a, b in pairs) / max(1, len(pairs)) if pairs else 0.0
        if multi:
            allp = [None] * n
            dist.all_gather_object(allp, local_us)
            local_us = max(allp)
        phases[name + "_us"] = round(local_us, 2)

    total_ms = reduce_max(times)
    ms_per_step = total_ms / args.steps
    if multi:
        alll = [None] * n
        dist.all_gather_object(alll, launches)
        launches = sum(alll)
    value = wire_bytes / (ms_per_step * 1e-3) / 1e9
    result = {
        "metric": "dispatch+combine aggregate wire GB/s (all ranks, max-over-ranks step time)",
        "value": round(value, 3),
        "unit": "GB/s",
        "n_gpus": n,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 5),
        "us_per_exchange": round(ms_per_step * 1e3, 2),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "fp8(e4m3)+bf16" if cfg.is_fp8 else "bf16",
        "data": "synthetic (seeded N(0,1) activations, distinct top-k routes, softmax weights; no weights involved)",
        "impl": args.impl,
        "config": {
            "model": f"AFD MoE exchange, BASELINE config {args.config}",
            "global_batch": T * attn,
            "seq_len": 1,
            "parallelism": f"{attn}A+{ffn}F" + (" colocated on one GPU" if not multi else ""),
            "hidden": cfg.hidden_size,
            "num_experts": cfg.num_experts,
            "top_k": cfg.top_k,
            "tokens_per_attention_rank": T,
            "payload": cfg.payload,
            "routing": "zipf(1.1)" if spec["zipf"] else "uniform",
            "l2": "flushed between steps (256 MiB fill)",
            "mode": "cuda-graph replay of complete exchanges (phases and e2e: eager launches)" if graph is not None else "eager",
            "wire_bytes_per_step": wire_bytes,
            "tokens_per_s": round(T * attn / (ms_per_step * 1e-3), 1),
            "per_attention_rank_GBs": round(value / attn, 3),
        },
        "expert_tflops": (
            round(6.0 * T * attn * cfg.top_k * cfg.hidden_size * spec["intermediate"] / (ms_per_step * 1e-3) / 1e12, 2)
            if "intermediate" in spec
            else None
        ),
        "expert_weights": (
            {"gate_up": args.expert_weights, "down": args.expert_down or args.expert_weights}
            if "intermediate" in spec
            else None
        ),
        "phases": phases,
        "roofline": dict(
            roofline,
            fraction_of_nvlink_roofline=round((roofline["dispatch_us_at_770GBs"] + roofline["combine_us_at_770GBs"]) / (ms_per_step * 1e3), 3),
        ),
        "clocks": clocks,
        "gpu_launches": launches,
        "wall_s_timed_region": round(t_wall1 - t_wall0, 3),
    }
    if e2e_times is not None:
        e2e_ms = reduce_max(e2e_times) / args.steps
        hi = sum(sum(t.numel() * t.element_size() for t in s["host"] if t is not None) for s in state if "host" in s)
        if multi:
            allh = [None] * n
            dist.all_gather_object(allh, hi)
            hi = sum(allh)
        result["e2e"] = {
            "value": round(wire_bytes / (e2e_ms * 1e-3) / 1e9, 3),
            "unit": "GB/s",
            "ms_per_step": round(e2e_ms, 5),
            "h2d_bytes_per_step": hi,
            "d2h_bytes_per_step": 4 * n,
        }
    if traces:
        names = ["dispatch", "receive", "reply", "collect"]
        lines = []
        for r, tr in traces:
            tr = tr.cpu()
            for k in range(4):
                t = tr[k]
                used = t[:, 0] > 0
                if not used.any():
                    continue
                t = t[used]
                s0 = int(t[:, 0].min())
                p1 = (int(t[:, 1].max()) - s0) / 1e3 if (t[:, 1] > 0).any() else float("nan")
                lines.append(
                    f"rank {r} {names[k]:9s} ctas={int(used.sum()):3d} start_ns={s0 % 10**9:9d} phase1_end={p1:7.1f}us "
                    f"first_cta_end={(int(t[:, 2].min()) - s0) / 1e3:7.1f}us last_cta_end={(int(t[:, 2].max()) - s0) / 1e3:7.1f}us"
                )
                if k in (0, 1) and (t[:, 3] >= s0).any():
                    col = t[:, 3][t[:, 3] >= s0]
                    what = "counts released" if k == 0 else "counts arrived"
                    lines.append(f"rank {r} {names[k]:9s} {what} at {(int(col.min()) - s0) / 1e3:.1f}..{(int(col.max()) - s0) / 1e3:.1f}us")
                # progress of warp 0's first record (receive) / token (collect) per CTA, min..max over CTAs
                detail = {1: (5, ("flag_seen", "landed", "stores_committed", "stores_complete")), 3: (6, ("flags_seen", "rows_landed", "stored"))}
                if k in detail and tr.shape[0] > detail[k][0]:
                    d = tr[detail[k][0]]
                    live = d[:, 0] >= s0
                    if live.any():
                        parts = []
                        for j, label in enumerate(detail[k][1]):
                            col = d[live][:, j]
                            col = col[col >= s0]
                            if col.numel():
                                parts.append(f"{label}={(int(col.min()) - s0) / 1e3:.1f}..{(int(col.max()) - s0) / 1e3:.1f}us")
                        lines.append(f"rank {r} {names[k]:9s} first item per CTA ({int(live.sum())} CTAs): " + " ".join(parts))
        if multi:
            alll = [None] * n
            dist.all_gather_object(alll, lines)
            lines = [l for part in alll for l in part]
        if rank == 0:
            print("\n".join(lines), file=sys.stderr)
    for s in state:
        s["buf"].check()
    if multi:
        buffers[0].close()
        dist.barrier()
        dist.destroy_process_group()
    else:
        world_obj.close()
    if rank == 0:
        print(json.dumps(result))


if __name__ == "__main__":
    main()
