// Grouped expert GEMM with the operands swapped: the expert's weight rows are the MMA's 128-row M
// operand and the tokens are a narrow N operand (64 columns), so a tile spends an eighth of the
// tensor time of the 128 x 256 kernel in grouped_gemm.cu per weight byte.  An alternative for
// batches of a few rows per expert, not the default: measured at 16 rows per expert (64 experts,
// FP8) the wide kernel already streams the weights at 4.8-5.6 TB/s and is 20-25 % faster than
// this one (0.336 vs 0.423 ms for 4096 x 7168 weights).  Same interface, same layouts:
//   out[r, :] = a[r, :] * W_e^T   for the rows r of expert e's segment,
// BF16 or block-scaled e4m3 operands, optional SwiGLU (gate/up rows of W alternate in blocks of
// 32) and routing weight.  Quantised (e4m3) output is not offered here: a 128-column scale group
// of the SwiGLU output spans two weight tiles.
//
// Layout of a CTA (persistent over work items = expert x 128 weight rows x 64 tokens):
//   warp 0      TMA producer: a 128 x BK tile of W and a 64 x BK tile of the activations per stage,
//               eight 24 KB stages deep (the kernel lives on memory latency)
//   warp 1      allocates tensor memory, one lane issues tcgen05.mma (M 128, N 64)
//   warps 2..5  epilogue: thread = TMEM lane = weight row = output column, 64 token values each.
//               FP8: every 128-deep K block lands in a fresh accumulator and is promoted with
//               a_scale[token] * w_scale.  SwiGLU: gate and up rows of a column pair sit in
//               different lane quarters, i.e. different warps; the "up" warp passes its values
//               through shared memory, tagged with the work item's number and acknowledged, so no
//               block-wide barrier is involved and every wait is bounded.
// The reference library has no GEMM; this is the small-batch expert path of the MoE layer.
#include <cuda_bf16.h>

#include "afdep/gemm_api.h"
#include "afdep/tcgen05.cuh"

namespace afdep {

namespace {

constexpr int BW = 128;                        // weight rows per tile (MMA M)
constexpr int NT = 64;                         // tokens per tile (MMA N)
constexpr int kStageBytes = (BW + NT) * 128;   // W tile + activation tile, 128-byte rows
constexpr int kStages = 8;
constexpr int kTmemCols = 128;                 // two NT-column fp32 accumulators
constexpr int kEpiWarps = 4;
constexpr int kThreads = (2 + kEpiWarps) * 32;
constexpr unsigned kSpinLimit = 1u << 28;      // probes before a wait gives up

struct Ctrl {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int failed;
    int tile_prefix[kMaxExpertsLocal + 1];     // work items of experts [0, e)
    int seg_start[kMaxExpertsLocal];
    int seg_rows[kMaxExpertsLocal];
    float up_vals[2][NT][32];                  // [column pair][token][lane]: "up" values on their way to the "gate" warp
    unsigned up_tag[2][32];                    // work item number + 1 whose values up_vals holds
    unsigned up_ack[2][32];                    // work item number + 1 the gate thread has consumed
};

__device__ __forceinline__ bool wait_bar(uint64_t* bar, unsigned parity, volatile int* failed) {
    for (unsigned i = 0; i < kSpinLimit; ++i) {
        if (ptx::mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *failed) return false;
    }
    *failed = 1;
    return false;
}

// Spin (bounded) until the shared-memory word equals `want`.
__device__ __forceinline__ bool wait_word(const volatile unsigned* word, unsigned want, volatile int* failed) {
    for (unsigned i = 0; i < kSpinLimit; ++i) {
        if (*word == want) return true;
        if ((i & 1023u) == 1023u && *failed) return false;
    }
    *failed = 1;
    return false;
}

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

template <bool kFp8>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_swapped_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                            const GroupedGemmArgs p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem + kStages * kStageBytes);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int BK = kFp8 ? 128 : 64;          // elements per 128-byte row
    const int num_kb = p.K / BK;
    const int n_tiles = p.N / BW;

    // ---- set-up ---------------------------------------------------------------------------
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(&ctrl->full[s], 1);
            ptx::mbar_init(&ctrl->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(&ctrl->acc_full[b], 1);
            ptx::mbar_init(&ctrl->acc_empty[b], kEpiWarps);
        }
        ctrl->failed = 0;
        ptx::fence_mbar_init();
        int run = 0, prev_end = 0;
        for (int e = 0; e < p.experts; ++e) {
            const int start = (prev_end + p.alignment - 1) / p.alignment * p.alignment;
            int end = p.ends[e];
            if (end > p.rows) end = p.rows;
            const int rows = end > start ? end - start : 0;
            ctrl->seg_start[e] = start;
            ctrl->seg_rows[e] = rows;
            ctrl->tile_prefix[e] = run;
            run += ((rows + NT - 1) / NT) * n_tiles;
            prev_end = p.ends[e];
        }
        ctrl->tile_prefix[p.experts] = run;
    }
    if (tid < 64) {
        (&ctrl->up_tag[0][0])[tid] = 0u;
        (&ctrl->up_ack[0][0])[tid] = 0u;
    }
    if (warp == 1) {
        tc::tmem_alloc(&ctrl->tmem_base, kTmemCols);
        tc::tmem_relinquish();
    }
    if (warp == 0 && lane == 0) {
        tc::prefetch_tensormap(&map_a);
        tc::prefetch_tensormap(&map_w);
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = ctrl->tmem_base;
    const int total_work = ctrl->tile_prefix[p.experts];
    volatile int* failed = &ctrl->failed;

    // Work item -> (expert, first weight row of the tile, first token row, live tokens).  Token
    // tiles of one weight tile are neighbours, then the weight tiles of one expert, so CTAs
    // working side by side share the small activation tile (and a re-read weight tile) in L2.
    auto decode = [&](int w, int& e, int& n0, int& tok0, int& live) {
        int lo = 0, hi = p.experts;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (ctrl->tile_prefix[mid] <= w) lo = mid; else hi = mid;
        }
        e = lo;
        const int local = w - ctrl->tile_prefix[e];
        const int t_tiles = (ctrl->tile_prefix[e + 1] - ctrl->tile_prefix[e]) / n_tiles;
        const int nt = local / t_tiles, tt = local - nt * t_tiles;
        n0 = nt * BW;
        tok0 = ctrl->seg_start[e] + tt * NT;
        live = ctrl->seg_rows[e] - tt * NT;
        if (live > NT) live = NT;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            unsigned phase = 0;
            for (int w = blockIdx.x; w < total_work; w += gridDim.x) {
                int e, n0, tok0, live;
                decode(w, e, n0, tok0, live);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!wait_bar(&ctrl->empty[stage], phase ^ 1u, failed)) break;
                    unsigned char* sw = smem + stage * kStageBytes;
                    ptx::mbar_expect_tx(&ctrl->full[stage], kStageBytes);
                    tc::tma_load_2d(sw, &map_w, kb * BK, e * p.N + n0, &ctrl->full[stage]);
                    tc::tma_load_2d(sw + BW * 128, &map_a, kb * BK, tok0, &ctrl->full[stage]);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (*failed) break;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = tc::instr_desc(BW, NT, kFp8 ? 0u : 1u, kFp8 ? 0u : 1u);
            constexpr int kMmaK = 32;            // bytes of K one instruction consumes
            int stage = 0;
            unsigned phase = 0;
            int acc_use = 0;
            for (int w = blockIdx.x; w < total_work && !*failed; w += gridDim.x) {
                for (int kb = 0; kb < num_kb; ++kb) {
                    const bool new_acc = kFp8 || kb == 0;
                    const int buf = acc_use & 1;
                    if (new_acc) {
                        if (!wait_bar(&ctrl->acc_empty[buf], ((acc_use >> 1) & 1u) ^ 1u, failed)) break;
                        tc::fence_after_sync();
                    }
                    if (!wait_bar(&ctrl->full[stage], phase, failed)) break;
                    tc::fence_after_sync();
                    const unsigned char* sw = smem + stage * kStageBytes;     // weights: the M operand
                    const unsigned char* sx = sw + BW * 128;                  // tokens: the N operand
                    const uint32_t d = tmem + (uint32_t)buf * NT;
#pragma unroll
                    for (int k = 0; k < 128 / kMmaK; ++k) {
                        const uint64_t da = tc::smem_desc_sw128(sw + k * kMmaK);
                        const uint64_t db = tc::smem_desc_sw128(sx + k * kMmaK);
                        const bool acc = kFp8 ? (k > 0) : (kb > 0 || k > 0);
                        if (kFp8)
                            tc::mma_fp8(d, da, db, idesc, acc);
                        else
                            tc::mma_bf16(d, da, db, idesc, acc);
                    }
                    tc::mma_commit(&ctrl->empty[stage]);
                    if (kFp8 || kb == num_kb - 1) {
                        tc::mma_commit(&ctrl->acc_full[buf]);
                        ++acc_use;
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps
        const int quarter = warp & 3;            // TMEM lanes [32 * quarter, +32) = weight rows of the tile
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const int pair = quarter >> 1;           // SwiGLU: which 32-column block of the output
        const bool is_up = (quarter & 1) != 0;   // SwiGLU: this warp holds "up" rows
        int acc_use = 0;
        unsigned item = 0;                       // work items this CTA has finished, the same in every warp
        for (int w = blockIdx.x; w < total_work && !*failed; w += gridDim.x, ++item) {
            int e, n0, tok0, live;
            decode(w, e, n0, tok0, live);
            // per-token factors live two per lane (tokens lane and lane + 32) and are broadcast by shuffle
            const int r_lo = min(tok0 + lane, p.rows - 1), r_hi = min(tok0 + 32 + lane, p.rows - 1);
            float acc[NT];
            bool ok = true;
            if (kFp8) {
#pragma unroll
                for (int t = 0; t < NT; ++t) acc[t] = 0.f;
                const float* a_lo = p.a_scale + (size_t)r_lo * p.a_scale_s0;
                const float* a_hi = p.a_scale + (size_t)r_hi * p.a_scale_s0;
                const float* w_sc = p.w_scale + ((size_t)e * (p.N / 128) + n0 / 128) * (p.K / 128);
                // scales are fetched one K block ahead: a global load must not sit between the
                // accumulator becoming ready and its promotion
                float s_lo_next = a_lo[0] * w_sc[0], s_hi_next = a_hi[0] * w_sc[0];
                for (int kb = 0; kb < num_kb; ++kb) {
                    const int buf = acc_use & 1;
                    const float s_lo = s_lo_next, s_hi = s_hi_next;
                    if (kb + 1 < num_kb) {
                        const float ws = w_sc[kb + 1];
                        s_lo_next = a_lo[(size_t)(kb + 1) * p.a_scale_s1] * ws;
                        s_hi_next = a_hi[(size_t)(kb + 1) * p.a_scale_s1] * ws;
                    }
                    if (!wait_bar(&ctrl->acc_full[buf], (acc_use >> 1) & 1u, failed)) {
                        ok = false;
                        break;
                    }
                    tc::fence_after_sync();
                    const uint32_t tsrc = tmem + lane_base + (uint32_t)(buf * NT);
                    uint32_t va[32], vb[32];
                    tc::tmem_ld32(tsrc, va);
                    tc::tmem_ld32(tsrc + 32u, vb);
                    tc::tmem_ld_wait_on(va);
                    tc::tmem_ld_wait_on(vb);
                    tc::fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&ctrl->acc_empty[buf]);     // the values are in registers
                    ++acc_use;
#pragma unroll
                    for (int t = 0; t < 32; ++t) {
                        acc[t] = fmaf(__uint_as_float(va[t]), __shfl_sync(ptx::kFullMask, s_lo, t), acc[t]);
                        acc[32 + t] = fmaf(__uint_as_float(vb[t]), __shfl_sync(ptx::kFullMask, s_hi, t), acc[32 + t]);
                    }
                }
                if (!ok) break;
            } else {
                const int buf = acc_use & 1;
                if (!wait_bar(&ctrl->acc_full[buf], (acc_use >> 1) & 1u, failed)) break;
                tc::fence_after_sync();
                const uint32_t tsrc = tmem + lane_base + (uint32_t)(buf * NT);
                uint32_t va[32], vb[32];
                tc::tmem_ld32(tsrc, va);
                tc::tmem_ld32(tsrc + 32u, vb);
                tc::tmem_ld_wait_on(va);
                tc::tmem_ld_wait_on(vb);
                tc::fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&ctrl->acc_empty[buf]);
                ++acc_use;
#pragma unroll
                for (int t = 0; t < 32; ++t) {
                    acc[t] = __uint_as_float(va[t]);
                    acc[32 + t] = __uint_as_float(vb[t]);
                }
            }

            // ---- output: this thread owns one output column, one value per token ---------------
            float rs_lo = 1.f, rs_hi = 1.f;
            if (p.row_scale != nullptr) {
                rs_lo = p.row_scale[r_lo];
                rs_hi = p.row_scale[r_hi];
            }
            if (p.swiglu) {
                if (is_up) {
                    // the gate thread must have taken the previous item's values out of the slot
                    if (!wait_word(&ctrl->up_ack[pair][lane], item, failed)) break;
#pragma unroll
                    for (int t = 0; t < NT; ++t) ctrl->up_vals[pair][t][lane] = acc[t];
                    __threadfence_block();
                    *reinterpret_cast<volatile unsigned*>(&ctrl->up_tag[pair][lane]) = item + 1u;
                } else {
                    if (!wait_word(&ctrl->up_tag[pair][lane], item + 1u, failed)) break;
                    __threadfence_block();
                    __nv_bfloat16* dst = p.out + (size_t)tok0 * p.ldc + n0 / 2 + pair * 32 + lane;
#pragma unroll
                    for (int t = 0; t < NT; ++t) {
                        const float up = *reinterpret_cast<volatile float*>(&ctrl->up_vals[pair][t][lane]);
                        const float rs = __shfl_sync(ptx::kFullMask, t < 32 ? rs_lo : rs_hi, t & 31);
                        if (t < live) dst[(size_t)t * p.ldc] = __float2bfloat16_rn(silu(acc[t]) * up * rs);
                    }
                    __threadfence_block();
                    *reinterpret_cast<volatile unsigned*>(&ctrl->up_ack[pair][lane]) = item + 1u;
                }
            } else {
                __nv_bfloat16* dst = p.out + (size_t)tok0 * p.ldc + n0 + quarter * 32 + lane;
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    const float rs = __shfl_sync(ptx::kFullMask, t < 32 ? rs_lo : rs_hi, t & 31);
                    if (t < live) dst[(size_t)t * p.ldc] = __float2bfloat16_rn(acc[t] * rs);
                }
            }
        }
    }

    // ---- teardown ---------------------------------------------------------------------------
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem, kTmemCols);
    }
    if (tid == 0 && ctrl->failed && p.error != nullptr) *p.error = 1;
}

constexpr int kSmemBytes = kStages * kStageBytes + (int)sizeof(Ctrl) + 1024;

}  // namespace

cudaError_t launch_grouped_gemm_swapped(const CUtensorMap& map_w, const CUtensorMap& map_a, const GroupedGemmArgs& args, int ctas,
                                        cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(grouped_gemm_swapped_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(grouped_gemm_swapped_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    if (args.fp8)
        grouped_gemm_swapped_kernel<true><<<ctas, kThreads, kSmemBytes, stream>>>(map_w, map_a, args);
    else
        grouped_gemm_swapped_kernel<false><<<ctas, kThreads, kSmemBytes, stream>>>(map_w, map_a, args);
    return cudaGetLastError();
}

}  // namespace afdep
