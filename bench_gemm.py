"""Micro-benchmark of the tcgen05 grouped expert GEMM against its roofline.

    python bench_gemm.py [--rows-per-expert 256] [--experts 64] [--n 4096] [--k 7168] [--dtype fp8|bf16] [--swiglu]
                         [--kernel promoting|selffeeding] [--gather]

``--kernel promoting`` is `grouped_gemm` (fp32 block scales promoted through registers),
``--kernel selffeeding`` is `expert_gemm` (power-of-two block scales applied by the tensor core;
``--gather`` reads the rows of A by index out of a shuffled matrix of records).

Times the kernel with CUDA events (warm-up, L2 flushed between iterations) and reports
achieved TFLOP/s next to the measured cuBLAS BF16 peak of `MEASURED_PEAKS.json` (FP8 is
reported against twice that figure) and, for reference, a cuBLAS BF16 matmul of the same shape
expert by expert.
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from afdep_b200.ops import grouped_gemm as gg


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--rows-per-expert", type=int, default=256)
    p.add_argument("--experts", type=int, default=64)
    p.add_argument("--n", type=int, default=4096)
    p.add_argument("--k", type=int, default=7168)
    p.add_argument("--dtype", choices=("fp8", "bf16"), default="fp8")
    p.add_argument("--swiglu", action="store_true")
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--ctas", type=int, default=0)
    p.add_argument("--skip-cublas", action="store_true")
    p.add_argument("--kernel", choices=("promoting", "selffeeding"), default="selffeeding")
    p.add_argument("--gather", action="store_true", help="self-feeding kernel: gather A rows by index from shuffled records")
    a = p.parse_args()
    torch.cuda.set_device(0)
    E, N, K, R = a.experts, a.n, a.k, a.rows_per_expert
    rows = E * ((R + 127) // 128 * 128)
    ends = torch.tensor([e * ((R + 127) // 128 * 128) + R for e in range(E)], dtype=torch.int32, device="cuda")
    x = torch.randn(rows, K, device="cuda") * 0.5
    w = torch.empty(E, N, K, device="cuda", dtype=torch.bfloat16)
    for e in range(E):
        w[e] = (torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16)
    kw = {}
    if a.dtype == "fp8":
        pow2 = a.kernel == "selffeeding"
        xa, a_scale = gg.quantize_rows_fp8(x, pow2)
        wq = torch.empty(E, N, K, device="cuda", dtype=torch.float8_e4m3fn)
        ws = torch.empty(E, N // 128, K // 128, device="cuda")
        for e in range(E):
            q, s = gg.quantize_weight_blocks_fp8(w[e : e + 1].float(), pow2)
            wq[e], ws[e] = q[0], s[0]
        wa, kw = wq, dict(a_scale=a_scale, w_scale=ws)
    else:
        xa, wa = x.to(torch.bfloat16), w
    out = torch.empty(rows, N // 2 if a.swiglu else N, device="cuda", dtype=torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    flops = 2.0 * E * R * N * K

    def timed(fn):
        ts = []
        for i in range(3 + a.iters):
            flush.fill_(i)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            if i >= 3:
                ts.append(e0.elapsed_time(e1))
        return sum(ts) / len(ts), min(ts)

    if a.kernel == "promoting":
        assert not a.gather, "--gather belongs to the self-feeding kernel"
        run = lambda: gg.grouped_gemm(xa, wa, ends, 128, swiglu=a.swiglu, out=out, ctas=a.ctas, **kw)      # noqa: E731
    elif a.gather:
        perm = torch.randperm(rows, device="cuda")
        index = torch.empty(rows, dtype=torch.int32, device="cuda")
        index[perm] = torch.arange(rows, dtype=torch.int32, device="cuda")           # row r lives in record index[r]
        if a.dtype == "fp8":
            rec_bytes = (K + (K // 128) * 4 + 127) // 128 * 128
            records = torch.zeros(rows, rec_bytes, dtype=torch.uint8, device="cuda")
            records[index.long(), :K] = xa.view(torch.uint8)
            records[index.long(), K : K + (K // 128) * 4] = kw["a_scale"].contiguous().view(torch.uint8).view(rows, -1)
            run = lambda: gg.expert_gemm(records, wa, ends, 128, swiglu=a.swiglu, out=out, ctas=a.ctas, w_scale=kw["w_scale"],      # noqa: E731
                                         row_index=index, a_scale_offset=K)
        else:
            records = torch.zeros(rows, K + 64, dtype=torch.bfloat16, device="cuda")
            records[index.long(), :K] = xa
            run = lambda: gg.expert_gemm(records, wa, ends, 128, swiglu=a.swiglu, out=out, ctas=a.ctas, row_index=index)             # noqa: E731
    else:
        run = lambda: gg.expert_gemm(xa, wa, ends, 128, swiglu=a.swiglu, out=out, ctas=a.ctas, **kw)        # noqa: E731
    mean_ms, best_ms = timed(run)
    torch.cuda.synchronize()
    assert not gg.gemm_check(), "a kernel gave up on a bounded wait"
    peaks = {}
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        peaks = json.load(open(path))
    bf16_peak = peaks.get("bf16_tflops", 1590.0)
    peak = bf16_peak * (2.0 if a.dtype == "fp8" else 1.0)
    res = {
        "kernel": "grouped_gemm" if a.kernel == "promoting" else "expert_gemm", "gather": a.gather, "dtype": a.dtype, "swiglu": a.swiglu, "experts": E, "rows_per_expert": R, "N": N, "K": K,
        "ms_mean": round(mean_ms, 4), "ms_best": round(best_ms, 4),
        "tflops_mean": round(flops / mean_ms / 1e9, 1), "tflops_best": round(flops / best_ms / 1e9, 1),
        "peak_tflops": peak, "peak_source": "measured cuBLAS bf16" + (" x2 for fp8" if a.dtype == "fp8" else "") if peaks else "fallback",
        "fraction_of_peak": round(flops / mean_ms / 1e9 / peak, 3),
        "weight_bytes": wa.numel() * wa.element_size(),
    }
    if not a.skip_cublas:
        xb = x.to(torch.bfloat16)
        step = (R + 127) // 128 * 128

        def cublas():
            for e in range(E):
                torch.matmul(xb[e * step : e * step + R], w[e].T)

        cm, cb = timed(cublas)
        res["cublas_bf16_per_expert_loop_ms"] = round(cm, 4)
        res["cublas_bf16_tflops"] = round(flops / cm / 1e9, 1)
    print(json.dumps(res))


if __name__ == "__main__":
    main()
