"""Headline benchmark: dispatch + combine of one AFD expert-parallel exchange.

    python bench.py --gpus N --steps K --warmup W [--impl ours|nccl|reference] [--config weak|2|3|4|5]

N = 1 runs one attention and one FFN rank colocated on a single GPU (all ranks in this
process); N >= 2 expects one process per GPU (torchrun) and splits the ranks N/2 FFN + N/2
attention (6 attention + 2 FFN for ``--config 4``).  A step is one complete exchange through
the public role API: ``source_dispatch`` -> ``worker_receive`` -> ``worker_reply`` ->
``source_collect``.  The FFN "expert" is the identity on a preallocated BF16 tensor, so the
timed region holds the library's four kernels and nothing else; ``--config 5`` puts SwiGLU
experts on tcgen05 in between (fused with the receive unless ``--unfused``).

Timing.  Every step is bracketed by CUDA events on the launching stream after a device-side
barrier across ranks (outside the events); L2 is flushed between steps.  K steps form a round;
rounds are repeated until the timed region spans at least 0.3 s, the round whose time is the
median supplies ``ms_per_step`` (maximum over ranks per round) and the spread is reported as
p10/p90.  ``value`` is the job's aggregate wire throughput: bytes that cross NVLink in both
directions (one record per token and destination FFN rank out, one BF16 row back) divided by
the step time; ``us_per_exchange`` and ``per_rank_GBs`` are the per-rank figures.  ``phases``
are kernel durations read from device time stamps of one traced graph replay.  The ``e2e``
entry repeats the measurement with, inside the timed region and every step, the host->device
copy of the step's inputs from pinned memory (one block per rank, one copy) and a device->host read of a checksum of the
result: ``serial`` issues the copy on the compute stream, the headline e2e ``value`` stages
step n+1's copy on a second stream while step n runs.  With ``--gpus 8`` the line also carries
sub-results for the 8-GPU configurations 3, 4 and 5 (5 both fused and as separate calls) under ``extra``.
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

# NVLink rate per direction per GPU: nominal, and what a bulk-copy kernel of this library reaches
# between two B200s of this pool (bench_nvlink.py; summary in profiles/nvlink_p2p_rate.md).
NVLINK_NOMINAL_GBS = 900.0
NVLINK_MEASURED_GBS = 770.0
MIN_TIMED_SECONDS = 0.3


def parse_args():
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=50)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", choices=("ours", "nccl", "reference"), default="ours")
    p.add_argument("--config", choices=tuple(CONFIGS), default="weak")
    p.add_argument("--expert-weights", choices=("fp8", "bf16"), default="fp8", help="config 5: storage of the expert weights")
    p.add_argument("--expert-down", choices=("fp8", "bf16"), default=None, help="config 5: storage of the down projection (default: like --expert-weights)")
    p.add_argument("--expert-scales", choices=("pow2", "fp32"), default="pow2",
                   help="config 5, FP8: block scales rounded up to powers of two and applied by the tensor core (default), or arbitrary fp32 scales promoted through registers")
    p.add_argument("--scale-format", choices=("fp32", "ue8m0x4"), default="fp32",
                   help="FP8 payloads: scales on the wire as fp32 (the reference's contract) or as packed exponent bytes")
    p.add_argument("--unfused", action="store_true", help="config 5: worker_receive -> experts -> worker_reply as separate calls")
    p.add_argument("--no-extra", action="store_true", help="--gpus 8: skip the sub-results for configs 3, 4 and 5")
    p.add_argument("--max-rounds", type=int, default=400, help="upper bound on the rounds of K steps (1 for a profiler capture)")
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


def percentile(values, q):
    v = sorted(values)
    if not v:
        return None
    pos = (len(v) - 1) * q
    lo = int(pos)
    hi = min(lo + 1, len(v) - 1)
    return v[lo] + (v[hi] - v[lo]) * (pos - lo)


class Env:
    """Process-wide state shared by the configurations measured in one invocation."""

    def __init__(self, args) -> None:
        import torch

        self.args, self.n = args, args.gpus
        self.multi = self.n > 1
        if self.multi:
            import datetime

            import torch.distributed as dist

            self.rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
            assert world == self.n, "launch with torchrun --nproc-per-node equal to --gpus"
            self.local = int(os.environ.get("LOCAL_RANK", self.rank))
            torch.cuda.set_device(self.local)
            dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=600))
        else:
            self.rank, self.local = 0, 0
            torch.cuda.set_device(0)
        self.dev = torch.device("cuda", self.local)
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.dev)

    def gather(self, obj):
        if not self.multi:
            return [obj]
        import torch.distributed as dist

        out = [None] * self.n
        dist.all_gather_object(out, obj)
        return out

    def host_barrier(self):
        if self.multi:
            import torch.distributed as dist

            dist.barrier()


def run_config(env: Env, name: str, *, steps: int, warmup: int, tokens: int = 0, with_e2e: bool = True, trace_print: bool = False,
               sampler: ClockSampler | None = None) -> dict:
    """Build the Buffers of one configuration, measure it, close them; returns the result record."""
    import torch

    from afdep_b200 import Buffer, Config
    from afdep_b200.utils import synthetic

    args, n, multi, dev = env.args, env.n, env.multi, env.dev
    spec = dict(CONFIGS[name])
    if tokens:
        spec["tokens"] = tokens
    ffn, attn = topology(n, name)
    T = spec["tokens"]
    experts_on = "intermediate" in spec
    pow2 = experts_on and args.expert_weights == "fp8" and (args.expert_down or "fp8") == "fp8" and args.expert_scales == "pow2"
    fused = experts_on and not args.unfused and args.impl == "ours" and (pow2 or args.expert_weights == "bf16")
    payload = spec["payload"]
    if experts_on and args.expert_weights == "bf16":
        payload = "bf16"
    packed = args.scale_format == "ue8m0x4" and payload == "fp8"
    cfg = Config(T, spec["hidden"], spec["experts_per_ffn"] * ffn, spec["top_k"], ffn, attn, payload=payload, num_sms=args.num_sms,
                 gpu_timeout_s=20, cpu_timeout_s=60, scale_format="ue8m0x4" if packed else "fp32")
    world_obj = None
    if multi:
        import torch.distributed as dist

        backend = "native" if args.impl == "ours" else "nccl"
        buffers = [Buffer(group=dist.group.WORLD, config=cfg, backend=backend)]
    else:
        from afdep_b200.parallel.loopback import LoopbackWorld

        world_obj = LoopbackWorld(cfg, gpu_timeout_s=20.0)
        buffers = world_obj.buffers

    # ---- per-rank state: pinned host inputs, two device input sets, expert weights ---------
    state = []
    for buf in buffers:
        s = {"buf": buf}
        if buf.role == "attention":
            x, ids, w, scale = synthetic.random_batch(cfg, T, seed=1000 + buf.role_rank, zipf_s=spec["zipf"], pow2_scales=pow2)
            # One pinned block holds a step's inputs back to back (256-byte aligned), and each of the
            # two device input sets is one block of the same shape: a step's inputs cross PCIe as one
            # copy instead of one per tensor.
            parts, offset = [], 0
            for t in (x, ids, w, scale):
                if t is None:
                    parts.append(None)
                    continue
                nbytes = t.numel() * t.element_size()
                parts.append((offset, nbytes, t.dtype, tuple(t.shape)))
                offset = (offset + nbytes + 255) // 256 * 256

            def views(block):
                return [None if q is None else block[q[0]:q[0] + q[1]].view(q[2]).view(q[3]) for q in parts]

            s["host_block"] = torch.empty(offset, dtype=torch.uint8).pin_memory()
            s["host"] = views(s["host_block"])
            for v, t in zip(s["host"], (x, ids, w, scale)):
                if t is not None:
                    v.copy_(t)
            s["dev_block"] = [s["host_block"].to(dev) for _ in range(2)]
            s["dev"] = [views(b) for b in s["dev_block"]]
            s["ids_cpu"] = ids
        elif experts_on:
            from afdep_b200.models.moe_layer import ExpertWeights

            s["weights"] = ExpertWeights.random(cfg.experts_per_rank, cfg.hidden_size, spec["intermediate"], mode=args.expert_weights,
                                                down=args.expert_down, seed=7 + buf.role_rank, device=dev,
                                                scale_format="pow2" if pow2 else "fp32")
        else:
            s["rows"] = torch.zeros((cfg.receive_rows(T), cfg.hidden_size), dtype=torch.bfloat16, device=dev)
        s["host_result"] = torch.zeros(1, dtype=torch.float32).pin_memory()
        state.append(s)

    # wire bytes per step (both directions) from the routes: one record per (token, FFN rank)
    el = cfg.experts_per_rank
    per_ffn = [0] * ffn
    egress = []
    for s in state:
        if "ids_cpu" in s:
            ids = s["ids_cpu"]
            dest = torch.where(ids >= 0, ids // el, torch.full_like(ids, -1))
            mine = [int((dest == f).any(dim=1).sum()) for f in range(ffn)]
            per_ffn = [p + m for p, m in zip(per_ffn, mine)]
            egress.append(sum(mine))
    gathered = env.gather((per_ffn, egress))
    per_ffn = [sum(g[0][f] for g in gathered) for f in range(ffn)]
    egress = [e for g in gathered for e in g[1]]
    records = sum(per_ffn)
    row_out = cfg.hidden_size * (1 if cfg.is_fp8 else 2) + (cfg.scale_groups * 4 if cfg.is_fp8 else 0)
    row_back = cfg.hidden_size * 2
    wire_bytes = records * (row_out + row_back)
    busiest = max(max(egress, default=0), max(per_ffn, default=0))

    ordered = sorted(state, key=lambda s: 0 if s["buf"].role == "attention" else 1)

    def barrier_all():
        if multi:
            if args.impl == "ours":
                buffers[0]._t._nb.barrier()
            else:
                import torch.distributed as dist

                dist.barrier()

    def step(which: int = 0):
        """One exchange in dependency order with input set ``which``; leaves a 1-element checksum
        of the rank's result in s["sum"]."""
        for s in ordered:
            if s["buf"].role == "attention":
                x, ids, w, scale = s["dev"][which]
                s["buf"].source_dispatch(x, ids, w, scale, bucket=T)
        for s in ordered:
            if s["buf"].role == "ffn":
                if experts_on and fused:
                    rec, _ = s["buf"].worker_serve_fused(s["weights"], bucket=T)
                else:
                    rec = s["buf"].worker_receive(bucket=T)
                    if experts_on:
                        from afdep_b200.models.moe_layer import run_experts

                        rows = run_experts(rec, s["weights"], cfg.expert_alignment)
                    else:
                        rows = rec.recv_x if not cfg.is_fp8 else s["rows"]
                    s["buf"].worker_reply(rows, rec.receipt)
                s["result"] = rec.recv_count_psum
        for s in ordered:
            if s["buf"].role == "attention":
                s["out"] = s["buf"].source_collect()
                s["result"] = s["out"]

    def read_back():
        """The step's result as the host sees it: a checksum per rank, copied to pinned memory."""
        for s in state:
            s["host_result"].copy_(s["result"].sum(dtype=torch.float32).reshape(1), non_blocking=True)

    def count_launches():
        return sum(int(s["buf"].stats().get("launches", 0)) for s in state)

    before_one = count_launches()
    step()
    torch.cuda.synchronize()
    launches_per_step = count_launches() - before_one
    env.host_barrier()

    # ---- CUDA graphs: one per input set, plus a traced one for the phase times ---------------
    use_graph = args.impl == "ours" and not args.eager
    side = torch.cuda.Stream()
    kernel_graph, graphs, traced_graph, traces = None, [None, None], None, []

    def capture(which, with_read_back):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            step(which)
            if with_read_back:
                read_back()
        return g

    if use_graph:
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                step()
        torch.cuda.synchronize()
        env.host_barrier()
        kernel_graph = capture(0, False)
        if with_e2e:
            graphs = [capture(0, True), capture(1, True)]
        traces = [(s["buf"].rank, s["buf"]._t._nb.trace(True)) for s in state]
        traced_graph = capture(0, False)
        for s in state:
            s["buf"]._t._nb.trace(False)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        env.host_barrier()

    def run_step(which=0):
        """A step as the end-to-end passes issue it: the exchange and the read-back of its result."""
        if graphs[which] is not None:
            graphs[which].replay()
        else:
            step(which)
            read_back()

    # ---- kernel-only timing: rounds of `steps` exchanges ---------------------------------------
    def timed_round(count):
        pairs = []
        for i in range(count):
            env.flush.fill_(i & 0xFF)
            barrier_all()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if kernel_graph is not None:
                kernel_graph.replay()
            else:
                step(0)
            e1.record()
            pairs.append((e0, e1))
        torch.cuda.synchronize()
        return [a.elapsed_time(b) for a, b in pairs]

    timed_round(warmup)
    if sampler is not None and env.rank == 0:
        sampler.start()
    t_wall0 = time.perf_counter()
    first = sum(timed_round(steps))
    # every rank must run the same number of rounds: agree on it from the slowest rank's first round
    first_max = max(env.gather(first))
    rounds = max(1, min(args.max_rounds, int(MIN_TIMED_SECONDS * 1e3 / max(first_max, 1e-3)) + 1))
    round_ms = [first] + [sum(timed_round(steps)) for _ in range(rounds - 1)]
    torch.cuda.synchronize()
    t_wall1 = time.perf_counter()
    samples_in_region = len(sampler.samples) if sampler is not None and env.rank == 0 else 0
    all_rounds = env.gather(round_ms)
    per_round = [max(r[i] for r in all_rounds) for i in range(len(round_ms))]      # max over ranks, round by round
    ms_per_step = percentile(per_round, 0.5) / steps
    launches = sum(env.gather(launches_per_step * steps * len(round_ms)))

    # ---- phases: kernel durations from one traced graph replay ------------------------------------
    phases, trace_lines = {}, []
    if traced_graph is not None:
        env.flush.fill_(1)
        barrier_all()
        traced_graph.replay()
        torch.cuda.synchronize()
        names = ["dispatch", "receive", "reply", "collect"]
        local_phase = {}
        for r, tr in traces:
            tr = tr.cpu()
            for k, kname in enumerate(names):
                t = tr[k]
                used = t[:, 0] > 0
                if not used.any():
                    continue
                t = t[used]
                s0 = int(t[:, 0].min())
                dur = (int(t[:, 2].max()) - s0) / 1e3
                local_phase[kname] = max(local_phase.get(kname, 0.0), dur)
                if trace_print:
                    p1 = (int(t[:, 1].max()) - s0) / 1e3 if (t[:, 1] > 0).any() else float("nan")
                    trace_lines.append(
                        f"rank {r} {kname:9s} ctas={int(used.sum()):3d} start_ns={s0 % 10**9:9d} phase1_end={p1:7.1f}us "
                        f"first_cta_end={(int(t[:, 2].min()) - s0) / 1e3:7.1f}us last_cta_end={dur:7.1f}us"
                    )
        for part in env.gather(local_phase):
            for kname, dur in part.items():
                phases[kname + "_us"] = round(max(phases.get(kname + "_us", 0.0), dur), 2)
        phases["source"] = "device time stamps of one traced graph replay: first CTA start to last CTA end of each kernel, maximum over ranks"
    if experts_on:
        # time of the FFN rank's part (receive + experts + reply) from events around it in an eager step
        ev = []
        for _ in range(3):
            env.flush.fill_(2)
            barrier_all()
            for s in ordered:
                if s["buf"].role == "attention":
                    x, ids, w, scale = s["dev"][0]
                    s["buf"].source_dispatch(x, ids, w, scale, bucket=T)
            for s in ordered:
                if s["buf"].role == "ffn":
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    if fused:
                        s["buf"].worker_serve_fused(s["weights"], bucket=T)
                    else:
                        from afdep_b200.models.moe_layer import run_experts

                        rec = s["buf"].worker_receive(bucket=T)
                        s["buf"].worker_reply(run_experts(rec, s["weights"], cfg.expert_alignment), rec.receipt)
                    b.record()
                    ev.append((a, b))
            for s in ordered:
                if s["buf"].role == "attention":
                    s["buf"].source_collect()
        torch.cuda.synchronize()
        local = min((a.elapsed_time(b) for a, b in ev), default=0.0) * 1e3
        phases["ffn_receive_experts_reply_us"] = round(max(env.gather(local)), 2)

    # ---- end to end: inputs from pinned host memory and a result read back, every step ----------
    e2e = None
    if with_e2e:
        copy_stream = torch.cuda.Stream()
        h2d = sum(s["host_block"].numel() for s in state if "host" in s)
        h2d = sum(env.gather(h2d))

        def copy_inputs(which, stream):
            with torch.cuda.stream(stream):
                for s in state:
                    if "host" in s:
                        s["dev_block"][which].copy_(s["host_block"], non_blocking=True)

        def e2e_serial(count):
            cur = torch.cuda.current_stream()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(count):
                copy_inputs(0, cur)
                run_step(0)
                cur.synchronize()               # the host reads the step's result before it issues the next step
            e1.record()
            e1.synchronize()
            return e0.elapsed_time(e1)

        def e2e_pipelined(count):
            cur = torch.cuda.current_stream()
            done = [torch.cuda.Event(), torch.cuda.Event()]       # input set filled
            free = [torch.cuda.Event(), torch.cuda.Event()]       # input set no longer read
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            copy_stream.wait_event(e0)
            copy_inputs(0, copy_stream)
            done[0].record(copy_stream)
            for i in range(count):
                b = i & 1
                cur.wait_event(done[b])
                if i + 1 < count:
                    if i >= 1:
                        copy_stream.wait_event(free[b ^ 1])
                    copy_inputs(b ^ 1, copy_stream)          # next step's inputs travel while this step runs
                    done[b ^ 1].record(copy_stream)
                run_step(b)
                free[b].record(cur)
                cur.synchronize()
            e1.record()
            e1.synchronize()
            return e0.elapsed_time(e1)

        for fn in (e2e_serial, e2e_pipelined):
            barrier_all()
            fn(max(3, warmup))
        e2e_rounds = max(1, min(rounds, 50))
        serial_ms, piped_ms = [], []
        for _ in range(e2e_rounds):
            barrier_all()
            torch.cuda.synchronize()
            serial_ms.append(e2e_serial(steps))
            barrier_all()
            torch.cuda.synchronize()
            piped_ms.append(e2e_pipelined(steps))
        serial = percentile([max(r[i] for r in env.gather(serial_ms)) for i in range(e2e_rounds)], 0.5) / steps
        piped = percentile([max(r[i] for r in env.gather(piped_ms)) for i in range(e2e_rounds)], 0.5) / steps
        e2e = {
            "value": round(wire_bytes / (piped * 1e-3) / 1e9, 3),
            "unit": "GB/s",
            "ms_per_step": round(piped, 5),
            "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": 4 * len(env.gather(0)) * (1 if multi else len(state)),
            "mode": "step n+1's inputs are copied on a second stream while step n runs; the host reads every step's checksum before issuing the next",
            "serial": {"value": round(wire_bytes / (serial * 1e-3) / 1e9, 3), "ms_per_step": round(serial, 5),
                       "mode": "copy, exchange and read-back back to back on one stream"},
            "rounds": e2e_rounds,
        }

    value = wire_bytes / (ms_per_step * 1e-3) / 1e9
    roof_900 = busiest * (row_out + row_back) / (NVLINK_NOMINAL_GBS * 1e9) * 1e6
    roof_meas = busiest * (row_out + row_back) / (NVLINK_MEASURED_GBS * 1e9) * 1e6
    result = {
        "metric": "dispatch+combine aggregate wire GB/s (all ranks, max-over-ranks step time)",
        "value": round(value, 3),
        "unit": "GB/s",
        "n_gpus": n,
        "steps": steps,
        "warmup": warmup,
        "ms_per_step": round(ms_per_step, 5),
        "us_per_exchange": round(ms_per_step * 1e3, 2),
        "per_rank_GBs": round(value / attn, 3),
        "rounds": len(per_round),
        "us_per_exchange_p10": round(percentile(per_round, 0.1) / steps * 1e3, 2),
        "us_per_exchange_p90": round(percentile(per_round, 0.9) / steps * 1e3, 2),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "fp8(e4m3)+bf16" if cfg.is_fp8 else "bf16",
        "data": "synthetic (seeded N(0,1) activations, distinct top-k routes, softmax weights" + ("; random-init N(0,0.02) expert weights)" if experts_on else "; no weights involved)"),
        "impl": args.impl,
        "config": {
            "model": f"AFD MoE exchange, config {name}",
            "global_batch": T * attn,
            "seq_len": 1,
            "parallelism": f"{attn}A+{ffn}F" + (" colocated on one GPU" if not multi else ""),
            "hidden": cfg.hidden_size,
            "num_experts": cfg.num_experts,
            "top_k": cfg.top_k,
            "tokens_per_attention_rank": T,
            "payload": cfg.payload,
            **({"scales_on_wire": cfg.scale_format} if cfg.is_fp8 else {}),
            "routing": "zipf(1.1)" if spec["zipf"] else "uniform",
            "l2": "flushed between steps (256 MiB fill); e2e: inputs arrive from host memory every step",
            "mode": "cuda-graph replay of complete exchanges" if use_graph else "eager",
            "wire_bytes_per_step": wire_bytes,
            "tokens_per_s": round(T * attn / (ms_per_step * 1e-3), 1),
        },
        "expert_tflops": (round(6.0 * T * attn * cfg.top_k * cfg.hidden_size * spec["intermediate"] / (ms_per_step * 1e-3) / 1e12, 2) if experts_on else None),
        "experts": (
            {"gate_up": args.expert_weights, "down": args.expert_down or args.expert_weights,
             "block_scales": ("powers of two, applied by the tensor core (deviation from plain amax/448 fp32 scales: each scale rounded up to 2^k)"
                              if pow2 else "fp32 amax/448, promoted through registers") if args.expert_weights == "fp8" else None,
             "fused_receive": fused}
            if experts_on else None
        ),
        "phases": phases,
        "roofline": {
            "busiest_port_records": busiest,
            "us_at_900GBs_nominal": round(roof_900, 2),
            "us_at_measured_rate": round(roof_meas, 2),
            "measured_rate_GBs": NVLINK_MEASURED_GBS,
            "fraction_at_900GBs_nominal": round(roof_900 / (ms_per_step * 1e3), 3),
            "fraction_at_measured_rate": round(roof_meas / (ms_per_step * 1e3), 3),
            "note": "colocated ranks share one GPU: no NVLink, HBM-bound" if not multi else "bytes through the busiest port, both directions",
        },
        "gpu_launches": launches,
        "wall_s_timed_region": round(t_wall1 - t_wall0, 3),
        "clock_samples_in_timed_region": samples_in_region,
    }
    if e2e is not None:
        result["e2e"] = e2e
    if trace_print and trace_lines:
        lines = [l for part in env.gather(trace_lines) for l in part]
        if env.rank == 0:
            print("\n".join(lines), file=sys.stderr)
    for s in state:
        s["buf"].check()
    graphs.clear()
    kernel_graph = traced_graph = None
    if multi:
        buffers[0].close()
    else:
        world_obj.close()
    env.host_barrier()
    return result


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    if args.gpus == 1 and args.impl != "ours":
        print(json.dumps({"impl": args.impl, "unavailable": "the NCCL baseline needs at least two ranks"}))
        return

    env = Env(args)
    sampler = ClockSampler(env.local)
    result = run_config(env, args.config, steps=args.steps, warmup=args.warmup, tokens=args.tokens, with_e2e=not args.no_e2e,
                        trace_print=args.trace, sampler=sampler)
    if env.n == 8 and args.config == "weak" and args.impl == "ours" and not args.no_extra:
        # the 8-GPU configurations, measured in the same run: skewed FP8 prefill, decode, end-to-end MoE layer
        extra = {}
        keys = ("value", "us_per_exchange", "us_per_exchange_p10", "us_per_exchange_p90", "per_rank_GBs", "rounds",
                "steps", "dtype", "config", "phases", "roofline", "expert_tflops", "experts", "gpu_launches")
        for name, k in (("3", 20), ("4", 100), ("5", 10)):
            sub = run_config(env, name, steps=k, warmup=3, with_e2e=False)
            extra["config" + name] = {key: sub[key] for key in keys}
        if not args.unfused:
            # the same MoE step with worker_receive -> experts -> worker_reply as separate calls, next to the fused one
            args.unfused = True
            try:
                sub = run_config(env, "5", steps=10, warmup=3, with_e2e=False)
            finally:
                args.unfused = False
            extra["config5_separate_calls"] = {key: sub[key] for key in keys}
        result["extra"] = extra
    # the sampler runs through every pass of this invocation: all of it is under load
    clocks = sampler.stop() if env.rank == 0 else None
    if clocks is not None:
        clocks["samples_in_device_timed_region"] = result.pop("clock_samples_in_timed_region", 0)
    result["clocks"] = clocks
    if env.multi:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    if env.rank == 0:
        print(json.dumps(result))


if __name__ == "__main__":
    main()
