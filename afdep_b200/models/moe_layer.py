"""An attention-FFN-disaggregated MoE layer on top of `Buffer`: the end-to-end use of the library.

Attention ranks hold tokens and a router decision; FFN ranks hold SwiGLU experts
(hidden -> intermediate -> hidden).  One layer step is

    attention:  source_dispatch(x, ids, weights)            ...            out = source_collect()
    FFN:                        worker_receive -> experts on tcgen05 -> worker_reply

The expert path is two grouped GEMMs (`afdep_b200.ops.grouped_gemm`):
  1. gate|up projection with SwiGLU in the epilogue.  With ``weights="fp8"`` the weights are
     stored e4m3 with one fp32 scale per 128 x 128 block and multiplied with e4m3 activations
     carrying per-row, per-128-column scales (block-scaled FP8, promotion in the epilogue);
  2. down projection with the routing weight applied to every output row.  With FP8 weights
     the first GEMM's epilogue quantises the SwiGLU output to e4m3 (one scale per row and 128
     columns), so the down projection is block-scaled FP8 as well and reads half the weight
     bytes; ``down="bf16"`` keeps the e4m3-rounded down weights in BF16 and the SwiGLU output
     in BF16 instead (the tensor cores do not mix BF16 and FP8 operands).

Two FP8 scale formats: ``scale_format="fp32"`` keeps arbitrary fp32 block scales (amax / 448;
every 128-deep K block is promoted through registers), ``scale_format="pow2"`` rounds every
scale up to a power of two so that the tensor core applies the scales itself
(``expert_gemm``; about twice the FP8 throughput, at most one bit of e4m3 range given up).
``serve(fused=True)`` additionally skips the expert-major copy of the received rows: the
gate|up GEMM gathers its rows straight from the wire records as their arrival flags land
(BF16 payload with BF16 experts, or FP8 payload with ``pow2`` FP8 experts).

The reference library stops at the exchange (its README leaves routing, quantization and
expert GEMMs to the caller); this module is the "caller" used by the end-to-end benchmark.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..buffer import Buffer, ReceiveResult
from ..ops import grouped_gemm as gg


@dataclass
class ExpertWeights:
    """Weights of the local experts of one FFN rank, in the layouts the kernels consume."""

    w_gate_up: torch.Tensor            # [E, 2I, H] bf16 or e4m3, gate/up interleaved in 32-row blocks
    w_gate_up_scale: torch.Tensor | None   # [E, 2I/128, H/128] fp32 (FP8 only)
    w_down: torch.Tensor               # [E, H, I] bf16, or e4m3 when w_down_scale is set
    intermediate: int
    mode: str
    w_down_scale: torch.Tensor | None = None   # [E, H/128, I/128] fp32 (FP8 down projection only)
    scale_format: str = "fp32"                 # "fp32": any fp32 block scale; "pow2": powers of two (hardware block scaling)

    @staticmethod
    def random(num_local_experts: int, hidden: int, intermediate: int, *, mode: str = "bf16", seed: int = 0, device="cuda", std: float = 0.02,
               down: str | None = None, scale_format: str = "fp32") -> "ExpertWeights":
        """Random-init N(0, std) experts; ``mode`` is "bf16" or "fp8" (e4m3 storage, 128 x 128 scales).
        ``down`` ("fp8" | "bf16", default: like ``mode``) picks the storage of the down projection;
        ``scale_format`` ("fp32" | "pow2") the form of the FP8 block scales."""
        assert mode in ("bf16", "fp8") and scale_format in ("fp32", "pow2")
        pow2 = scale_format == "pow2"
        assert not pow2 or (mode == "fp8" and (down or mode) == "fp8"), "power-of-two scales are an FP8 format (gate/up and down)"
        down = down or mode
        assert down in ("bf16", "fp8") and (down == "bf16" or mode == "fp8"), "an FP8 down projection needs FP8 gate/up weights"
        gen = torch.Generator(device=device).manual_seed(seed)
        E, I, H = num_local_experts, intermediate, hidden
        gate_up = torch.empty((E, 2 * I, H), device=device, dtype=torch.bfloat16)
        down_w = torch.empty((E, H, I), device=device, dtype=torch.bfloat16)
        for e in range(E):       # expert by expert: the fp32 staging stays small
            wg = torch.randn((I, H), generator=gen, device=device) * std
            wu = torch.randn((I, H), generator=gen, device=device) * std
            gate_up[e] = gg.interleave_gate_up(wg[None], wu[None])[0].to(torch.bfloat16)
            down_w[e] = (torch.randn((H, I), generator=gen, device=device) * std).to(torch.bfloat16)
        if mode == "bf16":
            return ExpertWeights(gate_up, None, down_w, I, mode)
        q = torch.empty((E, 2 * I, H), device=device, dtype=torch.float8_e4m3fn)
        scale = torch.empty((E, 2 * I // 128, H // 128), device=device, dtype=torch.float32)
        down_q = torch.empty((E, H, I), device=device, dtype=torch.float8_e4m3fn) if down == "fp8" else None
        down_scale = torch.empty((E, H // 128, I // 128), device=device, dtype=torch.float32) if down == "fp8" else None
        for e in range(E):
            qe, se = gg.quantize_weight_blocks_fp8(gate_up[e : e + 1].float(), pow2)
            q[e], scale[e] = qe[0], se[0]
            de, ds = gg.quantize_weight_blocks_fp8(down_w[e : e + 1].float(), pow2)
            if down == "fp8":
                down_q[e], down_scale[e] = de[0], ds[0]
            else:
                blocks = de.float().view(1, H // 128, 128, I // 128, 128) * ds.view(1, H // 128, 1, I // 128, 1)
                down_w[e] = blocks.reshape(H, I).to(torch.bfloat16)      # e4m3-rounded values, BF16 storage
        if down == "fp8":
            return ExpertWeights(q, scale, down_q, I, mode, down_scale, scale_format)
        return ExpertWeights(q, scale, down_w, I, mode)


def _fp32_scales(scale, hidden: int):
    """Received scales as fp32 [rows, hidden / 128]: packed exponent bytes (int32 words, from a
    Buffer with ``scale_format="ue8m0x4"``) are expanded, fp32 scales pass through."""
    if scale is not None and scale.dtype == torch.int32:
        from ..utils.scales import unpack_ue8m0x4

        return unpack_ue8m0x4(scale, hidden // 128)
    return scale


def run_experts(received: ReceiveResult, weights: ExpertWeights, alignment: int, *, scratch: dict | None = None) -> torch.Tensor:
    """BF16 rows for ``worker_reply``: SwiGLU MLP of every received row, times its routing weight."""
    x, ends = received.recv_x, received.recv_count_psum
    fp8 = weights.mode == "fp8"
    pow2 = weights.scale_format == "pow2"
    if fp8 and x.dtype != torch.float8_e4m3fn:
        # BF16 dispatch into FP8 experts: quantise the live rows on the FFN rank (one kernel)
        x, a_scale = gg.quantize_rows_fp8_cuda(x, ends[-1:], pow2)
    else:
        # packed exponent words go to the block-scaled kernel as they are; the promoting kernel wants fp32
        a_scale = received.recv_scale if pow2 else _fp32_scales(received.recv_scale, x.shape[1])
    if pow2:
        # hardware block scaling end to end: both GEMMs accumulate all of K in tensor memory
        h_q, h_scale = gg.expert_gemm(x, weights.w_gate_up, ends, alignment, swiglu=True, a_scale=a_scale,
                                      w_scale=weights.w_gate_up_scale, quantize_out=True)
        return gg.expert_gemm(h_q, weights.w_down, ends, alignment, row_scale=received.recv_topk_weights,
                              a_scale=h_scale, w_scale=weights.w_down_scale)
    if weights.w_down_scale is not None:
        h_q, h_scale = gg.grouped_gemm(x, weights.w_gate_up, ends, alignment, swiglu=True, a_scale=a_scale,
                                       w_scale=weights.w_gate_up_scale, quantize_out=True)
        return gg.grouped_gemm(h_q, weights.w_down, ends, alignment, row_scale=received.recv_topk_weights,
                               a_scale=h_scale, w_scale=weights.w_down_scale)
    h = gg.grouped_gemm(x, weights.w_gate_up, ends, alignment, swiglu=True, a_scale=a_scale if fp8 else None,
                        w_scale=weights.w_gate_up_scale)
    return gg.grouped_gemm(h, weights.w_down, ends, alignment, row_scale=received.recv_topk_weights)


def reference_experts(received: ReceiveResult, weights: ExpertWeights, alignment: int) -> torch.Tensor:
    """The same MLP in fp32 torch on the dequantised operands (test oracle)."""
    x, ends = received.recv_x, received.recv_count_psum
    fp8 = weights.mode == "fp8"
    a_scale = _fp32_scales(received.recv_scale, x.shape[1])
    pow2 = weights.scale_format == "pow2"
    if fp8 and x.dtype != torch.float8_e4m3fn:
        x, a_scale = gg.quantize_rows_fp8(x, pow2)
    h = gg.reference_grouped_gemm(x, weights.w_gate_up, ends.cpu(), alignment, swiglu=True, a_scale=a_scale if fp8 else None,
                                  w_scale=weights.w_gate_up_scale)
    if weights.w_down_scale is not None:
        h_q, h_scale = gg.quantize_rows_fp8(h, pow2)
        y = gg.reference_grouped_gemm(h_q, weights.w_down, ends.cpu(), alignment, row_scale=received.recv_topk_weights,
                                      a_scale=h_scale, w_scale=weights.w_down_scale)
        return y.to(torch.bfloat16)
    h = h.to(torch.bfloat16)
    y = gg.reference_grouped_gemm(h, weights.w_down, ends.cpu(), alignment, row_scale=received.recv_topk_weights)
    return y.to(torch.bfloat16)


class AfdMoELayer:
    """One MoE layer bound to a Buffer.  Attention ranks call ``forward``, FFN ranks ``serve``."""

    def __init__(self, buffer: Buffer, weights: ExpertWeights | None = None) -> None:
        self.buffer, self.config = buffer, buffer.config
        self.weights = weights
        if buffer.role == "ffn":
            assert weights is not None, "FFN ranks need expert weights"
            assert self.config.expert_alignment % 128 == 0, "the grouped GEMM needs expert_alignment to be a multiple of 128"

    def forward(self, x, ids, topk_weights, x_scale=None, *, bucket: int | None = None):
        """Attention rank: returns BF16 [T, H], each token's weighted expert outputs summed."""
        bucket = bucket or self.config.capacity_tokens_per_rank
        self.buffer.source_dispatch(x, ids, topk_weights, x_scale, bucket=bucket)
        return self.buffer.source_collect()

    def serve(self, *, bucket: int | None = None, fused: bool = False) -> ReceiveResult:
        """FFN rank: receive one exchange, run the local experts, reply.

        ``fused=True`` runs the sequence without materialising ``recv_x``: the gate|up GEMM reads
        its rows from the wire records as they arrive (``Buffer.worker_serve_fused``).  The returned
        ``ReceiveResult`` then has ``recv_x = None``.  It saves the receive pass and the memory of
        ``recv_x``; its row gather feeds the tensor cores more slowly than a tensor-map load, so
        measured on B200s it is level with the separate calls at decode sizes and a few per cent
        behind them once the gate|up GEMM is compute-bound (about 2,048 tokens per rank and up)."""
        bucket = bucket or self.config.capacity_tokens_per_rank
        if fused:
            received, _ = self.buffer.worker_serve_fused(self.weights, bucket=bucket)
            return received
        received = self.buffer.worker_receive(bucket=bucket)
        rows = run_experts(received, self.weights, self.config.expert_alignment)
        self.buffer.worker_reply(rows, received.receipt)
        return received
