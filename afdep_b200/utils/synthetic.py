"""Seeded synthetic inputs for tests and benchmarks (there are no datasets or checkpoints).

Two families:

* ``exact_batch`` — values chosen so that every product and sum of the synthetic expert
  (``row * (e + 1) * weight``) is exactly representable in BF16, and in e4m3 with power-of-two
  scales, so results can be compared bit for bit (the reference's GPU test does the same,
  tests/gpu/deepep.py:39-60).
* ``random_batch`` — N(0,1) activations, uniform or Zipf-skewed distinct top-k routes and
  softmax weights, the shapes the benchmark configurations name.
"""

from __future__ import annotations

import torch

from ..config import Config


def distinct_routes(tokens: int, num_experts: int, top_k: int, generator: torch.Generator, probs: torch.Tensor | None = None) -> torch.Tensor:
    """int64 [tokens, top_k]: top_k distinct experts per token, uniform or by ``probs``."""
    if tokens == 0:
        return torch.empty((0, top_k), dtype=torch.int64)
    if probs is None:
        scores = torch.rand((tokens, num_experts), generator=generator)
    else:
        # Gumbel top-k = sampling without replacement proportional to probs
        u = torch.rand((tokens, num_experts), generator=generator).clamp_(1e-12, 1 - 1e-12)
        scores = torch.log(probs)[None, :] - torch.log(-torch.log(u))
    return scores.topk(top_k, dim=1).indices.to(torch.int64)


def zipf_probs(num_experts: int, s: float, generator: torch.Generator) -> torch.Tensor:
    """Expert probabilities proportional to rank^-s over a seeded permutation of the experts."""
    ranks = torch.arange(1, num_experts + 1, dtype=torch.float64) ** (-s)
    perm = torch.randperm(num_experts, generator=generator)
    probs = torch.empty(num_experts, dtype=torch.float64)
    probs[perm] = ranks / ranks.sum()
    return probs.float()


def pow2_ceil(scale: torch.Tensor) -> torch.Tensor:
    """Positive fp32 values rounded up to powers of two (exact: mantissa and exponent are split,
    never a logarithm)."""
    mant, exp = torch.frexp(scale.float())               # scale = mant * 2^exp, mant in [0.5, 1)
    exp = exp - (mant == 0.5).to(exp.dtype)              # already a power of two: keep it
    return torch.ldexp(torch.ones_like(mant), exp)


def quantize_fp8(x: torch.Tensor, pow2: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """e4m3 rows with one fp32 scale per 128 channels (amax / 448; ``pow2`` rounds the scale up
    to a power of two, the form the hardware block-scaled expert GEMM takes)."""
    rows, hidden = x.shape
    g = x.float().view(rows, hidden // 128, 128)
    scale = (g.abs().amax(dim=2).double().clamp_min(1e-12) / 448.0).float()
    if pow2:
        scale = pow2_ceil(scale)
    q = (g / scale[:, :, None]).reshape(rows, hidden).to(torch.float8_e4m3fn)
    return q, scale


def _wire_scales(config: Config, scale: torch.Tensor) -> torch.Tensor:
    """fp32 scales in the form the configuration puts on the wire."""
    if config.scale_packed:
        from .scales import pack_ue8m0x4

        return pack_ue8m0x4(scale)
    return scale


def random_batch(config: Config, tokens: int, seed: int, *, zipf_s: float | None = None, skip_fraction: float = 0.0, pow2_scales: bool = False):
    """(x, ids, weights, x_scale) on the CPU for one attention rank."""
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn((tokens, config.hidden_size), generator=gen)
    probs = None
    if zipf_s is not None:
        probs = zipf_probs(config.num_experts, zipf_s, torch.Generator().manual_seed(1234))
    ids = distinct_routes(tokens, config.num_experts, config.top_k, gen, probs)
    logits = torch.randn((tokens, config.top_k), generator=gen)
    weights = torch.softmax(logits, dim=1).float()
    if skip_fraction > 0 and tokens:
        drop = torch.rand((tokens, config.top_k), generator=gen) < skip_fraction
        ids = torch.where(drop, torch.full_like(ids, -1), ids)
        weights = torch.where(drop, torch.zeros_like(weights), weights)
    if config.is_fp8:
        q, scale = quantize_fp8(x, pow2_scales or config.scale_packed)
        return q, ids, weights, _wire_scales(config, scale)
    return x.to(torch.bfloat16), ids, weights, None


def exact_batch(config: Config, tokens: int, source: int, epoch: int, *, active: int | None = None, routing: str = "mixed"):
    """Exactly representable inputs: signs from a (token, source, epoch) signature,
    magnitudes 2^(c % 4) / 16, weights 1/4 or 1/8, power-of-two FP8 scales."""
    H, K, E = config.hidden_size, config.top_k, config.num_experts
    t = torch.arange(tokens, dtype=torch.int64)
    col = torch.arange(H, dtype=torch.int64)
    sig = (t * 2654435761 + (source + 1) * 40503 + epoch * 9176) & 0xFFFFFF
    signs = (((sig[:, None] >> (col[None, :] % 24)) & 1) * 2 - 1).float()
    mags = (2.0 ** (col % 4).float()) / 16
    x = signs * mags
    slots = torch.arange(K, dtype=torch.int64)
    if routing == "skew":        # everything lands on the first FFN rank's experts
        el = config.experts_per_rank
        ids = (t[:, None] + slots[None, :]) % el
        ids = torch.where(slots[None, :] < el, ids, torch.full_like(ids, -1))
    else:                        # consecutive experts, rotating with token/source/epoch
        ids = (t[:, None] * 3 + slots[None, :] + source + epoch) % E
    weights = torch.full((tokens, K), 0.25 if K <= 4 else 0.125, dtype=torch.float32)
    live = t < (tokens if active is None else active)
    if routing == "skip":
        live = torch.zeros_like(live)
    ids = torch.where(live[:, None], ids, torch.full_like(ids, -1))
    weights = torch.where(live[:, None] & (ids >= 0), weights, torch.zeros_like(weights))
    if config.is_fp8:
        groups = torch.arange(H // 128)
        scale = (2.0 ** (groups % 3 - 1).float())[None, :].expand(tokens, -1).contiguous()
        q = (x.view(tokens, -1, 128) / scale[:, :, None]).reshape(tokens, H).to(torch.float8_e4m3fn)
        return q, ids, weights, _wire_scales(config, scale)
    return x.to(torch.bfloat16), ids, weights, None
