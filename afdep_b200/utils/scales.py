"""Scale words of an FP8 payload.

An FP8 row carries one scale per 128 channels.  The public contract is fp32; ``Config(...,
scale_format="ue8m0x4")`` carries the same scales as exponent bytes (UE8M0: the biased exponent
of a power-of-two fp32, nothing else), four to an int32 word in little-endian order, padded
with the exponent of 1.0.  That is the element the reference's native layer calls
``sf_pack_t.ue8m0x4`` (deep_ep/include/deep_ep/common/compiled.cuh:74-77) and the form in
which Blackwell's block-scaled MMA takes its scales; the exchange moves the words untouched.
"""

from __future__ import annotations

import torch

from ..config import Config

UE8M0_ONE = 127      # exponent byte of 1.0


def scale_dtype(config: Config) -> torch.dtype:
    """Element type of ``x_scale`` / ``recv_scale`` under ``config``."""
    return torch.int32 if config.scale_packed else torch.float32


def pack_ue8m0x4(scale: torch.Tensor) -> torch.Tensor:
    """fp32 power-of-two scales [rows, groups] -> int32 words [rows, ceil(groups / 4)].

    Raises if a scale is not a positive power of two: packing would change the value."""
    s = scale.float().contiguous()
    bits = s.view(torch.int32)
    if bool(((bits & 0x7FFFFF) != 0).any()) or bool((bits <= 0).any()):
        raise ValueError("UE8M0 packing needs positive power-of-two scales")
    rows, groups = s.shape
    words = (groups + 3) // 4
    expo = torch.full((rows, words * 4), UE8M0_ONE, dtype=torch.int32, device=s.device)
    expo[:, :groups] = (bits >> 23) & 0xFF
    expo = expo.view(rows, words, 4)
    # the top byte may set the sign bit of the word: assemble in int64 and narrow with wrap-around
    word = expo[:, :, 0].long() | (expo[:, :, 1].long() << 8) | (expo[:, :, 2].long() << 16) | (expo[:, :, 3].long() << 24)
    return ((word + (1 << 31)) % (1 << 32) - (1 << 31)).to(torch.int32)


def unpack_ue8m0x4(words: torch.Tensor, groups: int) -> torch.Tensor:
    """int32 words [rows, ceil(groups / 4)] (any strides) -> fp32 scales [rows, groups]."""
    w = words.contiguous().long() & 0xFFFFFFFF
    expo = torch.stack([(w >> (8 * b)) & 0xFF for b in range(4)], dim=-1).reshape(w.shape[0], -1)[:, :groups]
    return (expo.to(torch.int32) << 23).view(torch.float32)
