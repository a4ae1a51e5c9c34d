"""Deterministic routing layout of one source rank, as a stand-alone CUDA operation.

``route_layout(ids, num_experts, ffn_ranks)`` runs the first phase of the dispatch kernel on
its own and returns int32 tensors:

``route_e [T, K]``    the ids with ``-1`` kept and every choice of an illegal token set to ``-1``
``route_pos [T, K]``  how many earlier choices (token order, then k) of the same expert exist
``tok_slot [T, F]``   how many earlier tokens also send a record to FFN rank ``f``, or ``-1``
``counts [F + E]``    records per FFN rank, then choices per expert

``reference_layout`` is the same thing in plain torch, used to check the kernel.
"""

from __future__ import annotations

import torch

from ..utils import oracle


def route_layout(ids: torch.Tensor, num_experts: int, ffn_ranks: int):
    from .._native import load_native

    return load_native().route_layout(ids, int(num_experts), int(ffn_ranks))


def reference_layout(ids: torch.Tensor, num_experts: int, ffn_ranks: int):
    ids = oracle.legal_ids(ids.cpu(), num_experts)
    T, K = ids.shape
    el = num_experts // ffn_ranks
    pos = torch.full((T, K), -1, dtype=torch.int32)
    slot = torch.full((T, ffn_ranks), -1, dtype=torch.int32)
    counts = torch.zeros(ffn_ranks + num_experts, dtype=torch.int32)
    for t in range(T):
        seen = set()
        for k in range(K):
            e = int(ids[t, k])
            if e < 0:
                continue
            pos[t, k] = counts[ffn_ranks + e]
            counts[ffn_ranks + e] += 1
            seen.add(e // el)
        for f in sorted(seen):
            slot[t, f] = counts[f]
            counts[f] += 1
    return ids.to(torch.int32), pos, slot, counts
