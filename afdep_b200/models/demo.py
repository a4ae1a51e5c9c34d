"""A complete AFD MoE layer step, one process per rank: the smallest program that uses the library
the way a serving stack would.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \\
        -m afdep_b200.models.demo --ffn 2                       # 2 FFN + 2 attention GPUs
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \\
        -m afdep_b200.models.demo --ffn 2 --backend gloo        # the same on CPU (torch experts)

Attention ranks route random tokens (softmax top-k of random logits), FFN ranks run SwiGLU experts
on what they receive: the tcgen05 grouped GEMMs with the native backend, the fp32 torch
statement of the same MLP on CPU.  Every attention rank then checks its output against a dense
evaluation of the layer with the experts' weights rebuilt from their seeds, and rank 0 prints one
JSON line.  The reference library ships no such program: its README leaves routing and experts to
the caller.
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from ..buffer import Buffer
from ..config import Config
from .moe_layer import AfdMoELayer, ExpertWeights, reference_experts


def dense_layer(x: torch.Tensor, ids: torch.Tensor, w: torch.Tensor, experts: list[ExpertWeights], per_rank: int) -> torch.Tensor:
    """out[t] = sum_k w[t,k] * down_e(silu(gate_e x) * up_e x), e = ids[t,k], in fp32 on CPU."""
    xf = x.float().cpu()
    out = torch.zeros_like(xf)
    for e in sorted(set(ids[ids >= 0].tolist())):
        wt = experts[e // per_rank]
        le = e % per_rank
        gu = wt.w_gate_up[le].float().cpu()
        sel = (ids == e).cpu()
        tok = sel.any(dim=1)
        y = xf[tok] @ gu.T
        y = y.view(y.shape[0], -1, 2, 32)                      # gate / up interleaved in blocks of 32 rows
        h = (torch.nn.functional.silu(y[:, :, 0]) * y[:, :, 1]).reshape(y.shape[0], -1)
        o = h.to(torch.bfloat16).float() @ wt.w_down[le].float().cpu().T
        out[tok] += o * (w.cpu() * sel)[tok].sum(dim=1, keepdim=True)
    return out


def main(argv: list[str] | None = None) -> dict:
    import torch.distributed as dist

    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--ffn", type=int, default=0, help="FFN ranks (default: half of the job)")
    p.add_argument("--backend", choices=("native", "gloo"), default="native")
    p.add_argument("--tokens", type=int, default=64)
    p.add_argument("--hidden", type=int, default=512)
    p.add_argument("--intermediate", type=int, default=256)
    p.add_argument("--experts-per-rank", type=int, default=4)
    p.add_argument("--top-k", type=int, default=2)
    p.add_argument("--steps", type=int, default=2)
    a = p.parse_args(argv)

    own_group = not dist.is_initialized()
    if own_group:
        dist.init_process_group("gloo")                        # CPU control plane, owned by the caller
    rank, world = dist.get_rank(), dist.get_world_size()
    ffn = a.ffn or world // 2
    native = a.backend == "native"
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank))) if native else torch.device("cpu")
    if native:
        torch.cuda.set_device(device)
    cfg = Config(a.tokens, a.hidden, a.experts_per_rank * ffn, a.top_k, ffn, world - ffn, expert_alignment=128)
    buf = Buffer(group=dist.group.WORLD, config=cfg, backend=a.backend)

    def expert_weights(f: int, dev) -> ExpertWeights:
        # drawn on the CPU whatever the device: CPU and CUDA generators give different streams,
        # and the attention ranks rebuild every FFN rank's weights for their dense check
        wt = ExpertWeights.random(cfg.experts_per_rank, a.hidden, a.intermediate, mode="bf16", seed=100 + f, device="cpu")
        return ExpertWeights(wt.w_gate_up.to(dev), None, wt.w_down.to(dev), wt.intermediate, wt.mode)

    worst = 0.0
    if buf.role == "ffn":
        weights = expert_weights(buf.role_rank, device)
        layer = AfdMoELayer(buf, weights)
        for _ in range(a.steps):
            if native:
                layer.serve()
            else:                                              # CPU: the torch statement of the same experts
                rec = buf.worker_receive(bucket=a.tokens)
                buf.worker_reply(reference_experts(rec, weights, cfg.expert_alignment), rec.receipt)
    else:
        layer = AfdMoELayer(buf)
        everyone = [expert_weights(f, "cpu") for f in range(ffn)]
        gen = torch.Generator().manual_seed(7 + rank)
        for _ in range(a.steps):
            x = torch.randn(a.tokens, a.hidden, generator=gen).to(torch.bfloat16)
            logits = torch.randn(a.tokens, cfg.num_experts, generator=gen)
            top = logits.topk(a.top_k, dim=1)
            ids, w = top.indices.to(torch.int64), torch.softmax(top.values, dim=1)
            out = layer.forward(x.to(device), ids.to(device), w.to(device))
            want = dense_layer(x, ids, w, everyone, cfg.experts_per_rank)
            err = (out.float().cpu() - want).abs().max().item() / max(want.abs().max().item(), 1e-6)
            worst = max(worst, err)
    if native:
        torch.cuda.synchronize()
    buf.check()
    errors = [None] * world
    dist.all_gather_object(errors, worst)
    buf.close()
    result = {"ranks": world, "ffn_ranks": ffn, "backend": a.backend, "steps": a.steps, "max_relative_error": max(errors), "ok": max(errors) < 3e-2}
    if rank == 0:
        print(json.dumps(result))
    if own_group:
        dist.barrier()
        dist.destroy_process_group()
    if not result["ok"]:
        raise SystemExit(1)
    return result


if __name__ == "__main__":
    main()
