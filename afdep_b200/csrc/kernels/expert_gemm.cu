// Expert GEMM that feeds itself: C[rows, N] = A[rows, K] * W_e[N, K]^T over expert-major row
// segments, on tcgen05 with the accumulator in tensor memory.
//
// Roles of a CTA (persistent over 128 x 256 output tiles, 16 warps):
//   warp 0        tensor-map loads of the expert's 256 x BK weight tile (and of the 128 x BK tile
//                 of A in the dense form) into a ring of 128-byte-swizzled stages; in the gathered
//                 form it first waits until the tile's rows are all indexed and parks their record
//                 numbers in shared memory
//   warp 1        one lane issues tcgen05.mma (M 128, N 256) per stage and commits the stage-free,
//                 scale-slot-free and accumulator-ready mbarriers
//   warps 2-3     fused form only: index the exchange's wire records (poll the arrival flag, read
//                 the routing words, publish row -> record, weight, source; count rows per tile)
//   warps 4-7     feeders: gather the 128 rows of A with 16-byte asynchronous copies into the
//                 swizzled stage (gathered form), and write the scale exponents of four K blocks
//                 at a time into tensor memory (FP8 form; one warp per 32-lane quarter)
//   warps 8-15    epilogue: tcgen05.ld (thread = tile row, 128 columns per warp in two passes of
//                 64), SwiGLU / routing weight / BF16 or e4m3 output
//
// FP8 form (mx): kind::mxf8f6f4.block_scale.  The scales of the block-scaled format -- one per
// row and 128 columns of A, one per 128 x 128 block of W -- must be powers of two; their
// exponent bytes go to tensor memory (4 columns for A, 8 for W, per group of four K blocks, in a
// ring of four slots) and the tensor core applies them, so all of K accumulates in one
// 256-column accumulator and nothing is promoted through registers.  The MMAs of the next tile
// wait while the epilogue warps copy the accumulator out (about two of 56 K-block times).
// BF16 form: kind::f16, two 256-column accumulators in ping-pong.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "afdep/expert_gemm_api.h"
#include "afdep/ffn_layout.cuh"
#include "afdep/status.cuh"
#include "afdep/tcgen05.cuh"

namespace afdep {

namespace {

constexpr int BM = 128, BN = 256;
constexpr int kStages = 4;
constexpr int kStageBytes = (BM + BN) * 128;     // A tile + W tile, 128-byte rows
constexpr int kTmemCols = 512;
constexpr int kSfSlots = 4;                       // ring of scale groups (four K blocks each)
constexpr int kSfSlotCols = 16;                   // 4 columns for A's rows, 8 for W's, 4 spare
constexpr int kSfBase = BN;                       // scale slots follow the single FP8 accumulator
constexpr int kThreads = 512;
constexpr int kWarpIndex0 = 2, kIndexWarps = 2, kWarpFeed0 = 4, kFeedWarps = 4, kWarpEpi0 = 8, kEpiWarps = 8;
constexpr int kFeedThreads = kFeedWarps * 32;

struct Ctrl {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint64_t sf_full[kSfSlots];
    uint64_t sf_empty[kSfSlots];
    uint64_t rows_full[2];
    uint64_t rows_empty[2];
    uint32_t tmem_base;
    int failed;
    int tile_prefix[kMaxExpertsLocal + 1];
    int seg_start[kMaxExpertsLocal];
    int tile_rows[2][BM];                         // record number of every row of the tile being fed
    unsigned long long amax_x[2][2][BM];          // (tile number << 32 | row amax bits) per [parity][half][row]
};

// Bounded mbarrier wait: gives up after the clock budget, or as soon as another role has.
__device__ __forceinline__ bool wait_bar(uint64_t* bar, unsigned parity, volatile int* failed, long long budget) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (unsigned i = 1;; ++i) {
        if (ptx::mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 0) {
            if (*failed) return false;
            if (clock64() - t0 > budget) {
                *failed = 1;
                return false;
            }
        }
    }
}

// The same wait for a whole warp: one lane polls, all lanes learn the outcome together, so every
// exit from a role's loop is taken by complete warps (the loops contain warp-wide operations).
__device__ __forceinline__ bool wait_bar_warp(uint64_t* bar, unsigned parity, volatile int* failed, long long budget) {
    bool ok = true;
    if ((threadIdx.x & 31) == 0) ok = wait_bar(bar, parity, failed, budget);
    ok = __shfl_sync(ptx::kFullMask, ok, 0);
    __syncwarp();
    return ok;
}
__device__ __forceinline__ bool warp_dead(volatile int* failed) { return __shfl_sync(ptx::kFullMask, *failed, 0) != 0; }

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

__device__ __forceinline__ void red_release_gpu_add(unsigned* p, unsigned v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Smallest power of two >= m / 448, as a float and as its reciprocal (both exact).
__device__ __forceinline__ void pow2_scale(float m, float& scale, float& inv) {
    const unsigned bits = __float_as_uint(fmaxf(m, 1e-30f) * (1.f / 448.f));
    unsigned e = (bits >> 23) & 0xffu;
    if (bits & 0x7fffffu) ++e;
    e = min(max(e, 1u), 253u);
    scale = __uint_as_float(e << 23);
    inv = __uint_as_float((254u - e) << 23);
}

template <bool kMx, bool kGather>
__global__ void __launch_bounds__(kThreads, 1)
expert_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const ExpertGemmArgs p,
                   const FusedReceive fr) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem + kStages * kStageBytes);
    LayoutSmem* L = reinterpret_cast<LayoutSmem*>(reinterpret_cast<unsigned char*>(ctrl) + ((sizeof(Ctrl) + 15) & ~size_t(15)));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int BK = kMx ? 128 : 64;           // elements per 128-byte row
    constexpr int kAccBufs = kMx ? 1 : 2;
    const int num_kb = p.K / BK;
    const int n_tiles = (p.N + BN - 1) / BN;
    const bool fused = kGather && fr.enabled != 0;

    // ---- set-up -------------------------------------------------------------------------
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(&ctrl->full[s], kGather ? 1 + kFeedThreads : 1);
            ptx::mbar_init(&ctrl->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(&ctrl->acc_full[b], 1);
            ptx::mbar_init(&ctrl->acc_empty[b], kEpiWarps);
            ptx::mbar_init(&ctrl->rows_full[b], 1);
            ptx::mbar_init(&ctrl->rows_empty[b], kFeedWarps);
        }
        for (int s = 0; s < kSfSlots; ++s) {
            ptx::mbar_init(&ctrl->sf_full[s], kFeedWarps);
            ptx::mbar_init(&ctrl->sf_empty[s], 1);
        }
        ctrl->failed = 0;
        ptx::fence_mbar_init();
        int run = 0, prev_end = 0;
        for (int e = 0; e < p.experts; ++e) {
            const int start = (prev_end + p.alignment - 1) / p.alignment * p.alignment;
            const int end = p.ends[e];
            const int rows = end > start ? end - start : 0;
            ctrl->seg_start[e] = start;
            ctrl->tile_prefix[e] = run;
            run += ((rows + BM - 1) / BM) * n_tiles;
            prev_end = end;
        }
        ctrl->tile_prefix[p.experts] = run;
    }
    // The row-maximum mailboxes are matched by tile number, starting at 1: clear what an earlier
    // kernel on this SM left in shared memory, or a stale entry could pass for this launch's.
    for (int i = tid; i < 2 * 2 * BM; i += blockDim.x) (&ctrl->amax_x[0][0][0])[i] = 0ull;
    if (warp == 1) {
        tc::tmem_alloc(&ctrl->tmem_base, kTmemCols);
        tc::tmem_relinquish();
    }
    if (warp == 0 && lane == 0) {
        if (!kGather) tc::prefetch_tensormap(&map_a);
        tc::prefetch_tensormap(&map_w);
    }
    unsigned ep = 0;
    if (fused) {
        ep = ptx::ld_acquire_gpu(&fr.ws.epoch[0]) + 1u;
        load_layout(fr.c, fr.ws, *L);            // ends with a block barrier
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = ctrl->tmem_base;
    const int total_work = ctrl->tile_prefix[p.experts];
    volatile int* failed = &ctrl->failed;

    // Work item -> (expert, first row, first column); row tiles vary fastest inside an expert so
    // that CTAs working side by side share the expert's weight tile in L2.
    auto decode = [&](int w, int& e, int& row0, int& col0) {
        int lo = 0, hi = p.experts;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (ctrl->tile_prefix[mid] <= w) lo = mid; else hi = mid;
        }
        e = lo;
        const int local = w - ctrl->tile_prefix[e];
        const int m_tiles = (ctrl->tile_prefix[e + 1] - ctrl->tile_prefix[e]) / n_tiles;
        const int nt = local / m_tiles, mt = local - nt * m_tiles;
        row0 = ctrl->seg_start[e] + mt * BM;
        col0 = nt * BN;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        int stage = 0, tcount = 0;
        unsigned phase = 0;
        int next_rows[BM / 32];
        bool have_next = false;
        for (int w = blockIdx.x; w < total_work; w += gridDim.x) {
            int e, row0, col0;
            decode(w, e, row0, col0);
            if (kGather) {
                const int buf = tcount & 1;
                const int valid = min(BM, p.ends[e] - row0);
                bool ok = true;
                if (lane == 0) {
                    ok = wait_bar(&ctrl->rows_empty[buf], ((tcount >> 1) & 1u) ^ 1u, failed, p.budget);
                    if (ok && fused && !have_next) {
                        // every row of the tile has been indexed, i.e. all of its records have landed
                        const unsigned* cnt = fr.tile_cnt + (row0 >> 7);
                        const long long t0 = clock64();
                        unsigned it = 0;
                        while (ptx::ld_acquire_gpu(cnt) < (unsigned)valid) {
                            if ((++it & 63u) == 0 && (*failed || clock64() - t0 > p.budget)) {
                                *failed = 1;
                                ok = false;
                                break;
                            }
                        }
                    }
                }
                ok = __shfl_sync(ptx::kFullMask, ok, 0);
                __syncwarp();
                if (!ok) break;
#pragma unroll
                for (int j = 0; j < BM / 32; ++j) {
                    const int r = lane + 32 * j;
                    if (!have_next) next_rows[j] = (r < valid) ? __ldcg(p.row_rec + row0 + r) : -1;
                    ctrl->tile_rows[buf][r] = next_rows[j];
                }
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&ctrl->rows_full[buf]);
                ++tcount;
                // The row indices of this CTA's next tile are fetched now, so that their latency
                // passes while this tile's weights stream instead of holding up the next tile's
                // first loads.  In the fused form only a tile whose records have all been indexed
                // already is fetched ahead; any other waits for its counter when its turn comes.
                have_next = false;
                const int wn = w + (int)gridDim.x;
                if (wn < total_work) {
                    int en, rown, coln;
                    decode(wn, en, rown, coln);
                    const int validn = min(BM, p.ends[en] - rown);
                    bool ready = true;
                    if (fused) {
                        if (lane == 0) ready = ptx::ld_acquire_gpu(fr.tile_cnt + (rown >> 7)) >= (unsigned)validn;
                        ready = __shfl_sync(ptx::kFullMask, ready, 0);
                        __syncwarp();
                    }
                    if (ready) {
#pragma unroll
                        for (int j = 0; j < BM / 32; ++j) {
                            const int r = lane + 32 * j;
                            next_rows[j] = (r < validn) ? __ldcg(p.row_rec + rown + r) : -1;
                        }
                        have_next = true;
                    }
                }
            }
            if (lane == 0) {
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!wait_bar(&ctrl->empty[stage], phase ^ 1u, failed, p.budget)) break;
                    unsigned char* sa = smem + stage * kStageBytes;
                    ptx::mbar_expect_tx(&ctrl->full[stage], kGather ? BN * 128 : kStageBytes);
                    if (!kGather) tc::tma_load_2d(sa, &map_a, kb * BK, row0, &ctrl->full[stage]);
                    tc::tma_load_2d(sa + BM * 128, &map_w, kb * BK, e * p.N + col0, &ctrl->full[stage]);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            stage = __shfl_sync(ptx::kFullMask, stage, 0);
            phase = __shfl_sync(ptx::kFullMask, phase, 0);
            if (warp_dead(failed)) break;
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_bf16 = tc::instr_desc(BM, BN, 1u, 1u);
            constexpr int kMmaK = 32;            // bytes of K one instruction consumes
            int stage = 0;
            unsigned phase = 0;
            int acc_use = 0;
            unsigned group = 0;                  // scale groups consumed so far
            for (int w = blockIdx.x; w < total_work && !*failed; w += gridDim.x) {
                const int buf = acc_use % kAccBufs;
                if (!wait_bar(&ctrl->acc_empty[buf], ((acc_use / kAccBufs) & 1u) ^ 1u, failed, p.budget)) break;
                tc::fence_after_sync();
                const uint32_t d = tmem + (uint32_t)buf * BN;
                bool ok = true;
                for (int kb = 0; kb < num_kb; ++kb) {
                    const unsigned slot = group % kSfSlots;
                    if (kMx && (kb & 3) == 0) {
                        if (!wait_bar(&ctrl->sf_full[slot], (group / kSfSlots) & 1u, failed, p.budget)) {
                            ok = false;
                            break;
                        }
                    }
                    if (!wait_bar(&ctrl->full[stage], phase, failed, p.budget)) {
                        ok = false;
                        break;
                    }
                    tc::fence_after_sync();
                    const unsigned char* sa = smem + stage * kStageBytes;
                    const unsigned char* sb = sa + BM * 128;
                    const uint32_t sfa = tmem + (uint32_t)(kSfBase + slot * kSfSlotCols);
                    const uint32_t idesc_mx = tc::instr_desc_block_scaled(BM, BN, (uint32_t)(kb & 3), (uint32_t)(kb & 3));
#pragma unroll
                    for (int k = 0; k < 128 / kMmaK; ++k) {
                        const uint64_t da = tc::smem_desc_sw128(sa + k * kMmaK);
                        const uint64_t db = tc::smem_desc_sw128(sb + k * kMmaK);
                        const bool acc = kb > 0 || k > 0;
                        if (kMx)
                            tc::mma_mxfp8(d, da, db, idesc_mx, acc, sfa, sfa + 4);
                        else
                            tc::mma_bf16(d, da, db, idesc_bf16, acc);
                    }
                    tc::mma_commit(&ctrl->empty[stage]);
                    if (kMx && ((kb & 3) == 3 || kb == num_kb - 1)) {
                        tc::mma_commit(&ctrl->sf_empty[slot]);
                        ++group;
                    }
                    if (kb == num_kb - 1) tc::mma_commit(&ctrl->acc_full[buf]);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                ++acc_use;
            }
        }
    } else if (warp < kWarpFeed0) {
        // ------------------------------------------------------------------ record indexing
        if (fused) {
            const Geometry& g = fr.c.g;
            const int A = g.attn, K = g.top_k, EL = g.experts_local, C = g.capacity, fi = fr.c.role_rank;
            const WaitCtx wc{fr.c.status, fr.c.poison, fr.c.budget, fr.c.rank, /*kernel=*/12};
            const unsigned char* heap = reinterpret_cast<const unsigned char*>(fr.c.peer[fr.c.rank]);
            const uint32_t* slot_flag = reinterpret_cast<const uint32_t*>(heap + g.f_slot_flag);
            const unsigned char* stage_base = heap + g.f_stage;
            const int total = L->rec_prefix[A];
            const int G = gridDim.x;
            for (int item = (warp - kWarpIndex0) * G + blockIdx.x; item < total; item += kIndexWarps * G) {
                int a, slot;
                locate_striped(*L, A, item, a, slot);
                bool ok = true;
                if (lane == 0) {
                    const uint32_t* flag = slot_flag + (size_t)a * C + slot;
                    uint32_t seen = 0;
                    ok = spin_until(wc, [&] {
                        seen = ptx::ld_acquire_sys(flag);
                        return seen == ep;
                    });
                    if (!ok) {
                        report(wc, kTimeoutRecord, g.ffn + a, ep, ep, seen, slot, total);
                        poison(wc);
                        *failed = 1;
                    }
                    if (*failed) ok = false;
                }
                ok = __shfl_sync(ptx::kFullMask, ok, 0);
                __syncwarp();
                if (!ok) break;
                const int* meta = reinterpret_cast<const int*>(stage_base + ((size_t)a * C + slot) * g.rec_bytes + g.meta_off);
                const int src_token = __ldcg(meta + 3 * K);
                if (lane < K) {
                    const int e = __ldcg(meta + lane);
                    const int el = e - fi * EL;
                    if (e >= 0 && el >= 0 && el < EL) {
                        const int row = L->row_base[a * EL + el] + __ldcg(meta + K + lane);
                        if (row < 0 || row >= fr.rows_cap) {
                            report(wc, kBadIndex, g.ffn + a, ep, fr.rows_cap, row, slot, 4);
                        } else {
                            fr.row_rec[row] = a * C + slot;
                            fr.recv_w[row] = __int_as_float(__ldcg(meta + 2 * K + lane));
                            fr.recv_src[2 * (size_t)row] = a;
                            fr.recv_src[2 * (size_t)row + 1] = src_token;
                            red_release_gpu_add(fr.tile_cnt + (row >> 7), 1u);
                        }
                    }
                }
            }
        }
    } else if (warp < kWarpEpi0) {
        // ------------------------------------------------------------------ feeders
        const int ft = tid - kWarpFeed0 * 32;            // 0..127
        const int quarter = warp & 3;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        int stage = 0, tcount = 0;
        unsigned phase = 0, group = 0;
        for (int w = blockIdx.x; w < total_work && !warp_dead(failed); w += gridDim.x) {
            int e, row0, col0;
            decode(w, e, row0, col0);
            int rec_a[8], rec_s[4];
            const unsigned char* src_a[8];
            if (kGather) {
                const int buf = tcount & 1;
                if (!wait_bar_warp(&ctrl->rows_full[buf], (tcount >> 1) & 1u, failed, p.budget)) break;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    rec_a[i] = ctrl->tile_rows[buf][i * 16 + (ft >> 3)];
                    src_a[i] = p.a_rows + (size_t)(rec_a[i] >= 0 ? rec_a[i] : 0) * p.a_pitch + (ft & 7) * 16;
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) rec_s[j] = ctrl->tile_rows[buf][32 * j + lane];
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&ctrl->rows_empty[buf]);
                ++tcount;
            }
            const int row_limit = min(p.ends[e], p.rows);
            // Scales of one group (four K blocks): four rows per lane for A, two 128-column blocks for W.
            // They are fetched one group ahead, so their latency never holds up the row gathering.
            float sa[4][4], sb[2][4];
            uint32_t pa[4];                              // packed form: one word per row holds the group's four exponent bytes
            const bool a_packed = kMx && p.a_scale_packed != 0;
            const int kgroups = p.K / 128;
            const bool from_records = kGather && p.a_scale == nullptr;
            const float4* rec_scale[4];                  // gathered rows: the scales sit in the record, behind the payload
#pragma unroll
            for (int j = 0; j < 4; ++j)
                rec_scale[j] = (from_records && rec_s[j] >= 0)
                                   ? reinterpret_cast<const float4*>(p.a_rows + (size_t)rec_s[j] * p.a_pitch + p.a_scale_off)
                                   : nullptr;
            const float* w_scale0 = kMx ? p.w_scale + ((size_t)e * (p.N / 128) + col0 / 128) * kgroups : nullptr;
            const bool w_second = col0 + 128 < p.N;      // the tile's second 128-column block exists
            // groups of four scales are 16-byte aligned
            const bool w_vec = (kgroups & 3) == 0 && (reinterpret_cast<uintptr_t>(p.w_scale) & 15) == 0;
            auto fetch_scales = [&](int kb0) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int r = 32 * j + lane;
                    if (a_packed) {
                        uint32_t word = 0x7f7f7f7fu;             // four times the exponent of 1.0
                        if (from_records) {
                            if (rec_scale[j] != nullptr) word = __ldcg(reinterpret_cast<const uint32_t*>(rec_scale[j]) + (kb0 >> 2));
                        } else if (row0 + r < row_limit) {
                            word = __ldg(reinterpret_cast<const uint32_t*>(p.a_scale) + (size_t)(row0 + r) * p.a_scale_s0 +
                                         (size_t)(kb0 >> 2) * p.a_scale_s1);
                        }
                        pa[j] = word;
                    } else if (from_records) {
                        float4 v = make_float4(1.f, 1.f, 1.f, 1.f);
                        if (rec_scale[j] != nullptr) v = __ldcg(rec_scale[j] + (kb0 >> 2));
                        sa[j][0] = v.x;
                        sa[j][1] = v.y;
                        sa[j][2] = v.z;
                        sa[j][3] = v.w;
                    } else {
#pragma unroll
                        for (int b = 0; b < 4; ++b)
                            sa[j][b] = (kb0 + b < num_kb && row0 + r < row_limit)
                                           ? __ldg(p.a_scale + (size_t)(row0 + r) * p.a_scale_s0 + (size_t)(kb0 + b) * p.a_scale_s1)
                                           : 1.f;
                    }
                }
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const float* src = w_scale0 + (size_t)h * kgroups + kb0;
                    if (h == 1 && !w_second) {
#pragma unroll
                        for (int b = 0; b < 4; ++b) sb[h][b] = 1.f;
                    } else if (w_vec) {
                        const float4 v = __ldg(reinterpret_cast<const float4*>(src));
                        sb[h][0] = v.x;
                        sb[h][1] = v.y;
                        sb[h][2] = v.z;
                        sb[h][3] = v.w;
                    } else {
#pragma unroll
                        for (int b = 0; b < 4; ++b) sb[h][b] = (kb0 + b < num_kb) ? __ldg(src + b) : 1.f;
                    }
                }
            };
            // One scale group (four K blocks) takes four steps: pack the rows' scales into exponent
            // bytes; pack the columns' and start fetching the group after; store the bytes to TMEM once
            // the slot is free; wait for the stores and publish the slot.  The steps are spread over
            // the stages of the group BEFORE, one after each stage's copies have gone out, so that no
            // stage's copies start late by a whole group's work: a ring of four stages would delay the
            // same stage every time round, and the MMAs would wait for it every time.
            uint32_t wa[4], wb[2];
            auto pack_rows = [&](int kb0) {
                const bool whole = kb0 + 4 <= num_kb;
                if (a_packed) {                          // bytes past the last K block are never read by an MMA
#pragma unroll
                    for (int j = 0; j < 4; ++j) wa[j] = pa[j];
                    return;
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t word = 0;
#pragma unroll
                    for (int b = 0; b < 4; ++b) word |= ((whole || kb0 + b < num_kb) ? tc::ue8m0_of_pow2(sa[j][b]) : 127u) << (8 * b);
                    wa[j] = word;
                }
            };
            auto pack_cols = [&](int kb0) {                  // and start on the group after: both arrays are free now
                const bool whole = kb0 + 4 <= num_kb;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t word = 0;
#pragma unroll
                    for (int b = 0; b < 4; ++b) word |= ((whole || kb0 + b < num_kb) ? tc::ue8m0_of_pow2(sb[h][b]) : 127u) << (8 * b);
                    wb[h] = word;
                }
                if (kb0 + 4 < num_kb) fetch_scales(kb0 + 4);
            };
            auto store = [&]() -> bool {
                const unsigned slot = group % kSfSlots;
                if (!wait_bar_warp(&ctrl->sf_empty[slot], ((group / kSfSlots) & 1u) ^ 1u, failed, p.budget)) return false;
                tc::fence_after_sync();
                const uint32_t dst = tmem + lane_base + (uint32_t)(kSfBase + slot * kSfSlotCols);
                uint32_t wide[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) wide[j] = wb[j >> 2];
                tc::tmem_st4(dst, wa[0], wa[1], wa[2], wa[3]);
                tc::tmem_st8(dst + 4, wide);
                return true;
            };
            auto publish = [&]() {
                tc::tmem_st_wait();
                tc::fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&ctrl->sf_full[group % kSfSlots]);
                ++group;
            };
            if (kMx) fetch_scales(0);
            bool ok = true;
            for (int kb = 0; kb < num_kb && ok; ++kb) {
                if (kGather) {
                    if (!wait_bar_warp(&ctrl->empty[stage], phase ^ 1u, failed, p.budget)) {
                        ok = false;
                        break;
                    }
                    unsigned char* dst_a = smem + stage * kStageBytes;
                    const int chunk = ft & 7;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int r = i * 16 + (ft >> 3);
                        tc::cp_async16(dst_a + r * 128 + ((chunk ^ (r & 7)) << 4), src_a[i] + (size_t)kb * 128, rec_a[i] >= 0 ? 16u : 0u);
                    }
                    tc::cp_async_arrive(&ctrl->full[stage]);
                }
                if (kMx) {
                    const int g = kb >> 2, step = kb & 3, next = 4 * g + 4;
                    if (kb == 0) {                       // the tile's first group, all at once
                        pack_rows(0);
                        pack_cols(0);
                        ok = store();
                        if (ok) publish();
                    } else if (next < num_kb) {          // group g + 1 during group g
                        if (step == 0) pack_rows(next);
                        if (step == 1) {
                            if (g == 0) pack_rows(next);     // stage 0 was busy with the first group
                            pack_cols(next);
                        }
                        if (step == 2) ok = store();
                        if (step == 3) publish();
                    }
                }
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            if (!ok) break;
        }
        if (kGather) asm volatile("cp.async.wait_all;" ::: "memory");
    } else {
        // ------------------------------------------------------------------ epilogue
        const int quarter = warp & 3;
        const int half = (warp - kWarpEpi0) >> 2;            // which 128 columns of the tile
        const int r_in_tile = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        int acc_use = 0;
        unsigned tile_no = 0;
        for (int w = blockIdx.x; w < total_work && !warp_dead(failed); w += gridDim.x, ++tile_no) {
            int e, row0, col0;
            decode(w, e, row0, col0);
            const int hcol0 = col0 + half * 128;
            const bool half_ok = hcol0 < p.N;
            const int row = row0 + r_in_tile;
            const bool row_ok = row < p.ends[e] && row < p.rows && half_ok;
            const int buf = acc_use % kAccBufs;
            if (!wait_bar_warp(&ctrl->acc_full[buf], (acc_use / kAccBufs) & 1u, failed, p.budget)) break;
            tc::fence_after_sync();
            const float rs = (p.row_scale != nullptr && row_ok) ? p.row_scale[row] : 1.f;
            const uint32_t tbase = tmem + lane_base + (uint32_t)(buf * BN + half * 128);
            const bool quant = kMx && p.swiglu && p.out_q != nullptr;
            float hval[64];                      // SwiGLU outputs kept for the quantising epilogue
            float amax = 0.f;
#pragma unroll
            for (int pass = 0; pass < 2; ++pass) {
                uint32_t v0[32], v1[32];
                tc::tmem_ld32(tbase + (uint32_t)(pass * 64), v0);
                tc::tmem_ld32(tbase + (uint32_t)(pass * 64 + 32), v1);
                tc::tmem_ld_wait_on(v0);
                tc::tmem_ld_wait_on(v1);
                if (pass == 1) {
                    // the accumulator is in registers: hand it back before the arithmetic and the stores
                    tc::fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&ctrl->acc_empty[buf]);
                }
                if (p.swiglu) {
                    // 32 gate columns followed by their 32 up columns
                    if (quant) {
#pragma unroll
                        for (int c = 0; c < 32; ++c) {
                            const float h = silu(__uint_as_float(v0[c])) * __uint_as_float(v1[c]) * rs;
                            hval[pass * 32 + c] = h;
                            amax = fmaxf(amax, fabsf(h));
                        }
                    } else if (row_ok) {
                        __nv_bfloat16* dst = p.out + (size_t)row * p.ldc + hcol0 / 2 + pass * 32;
#pragma unroll
                        for (int c = 0; c < 32; c += 8) {
                            uint4 pk;
                            __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                q[i] = __floats2bfloat162_rn(silu(__uint_as_float(v0[c + 2 * i])) * __uint_as_float(v1[c + 2 * i]) * rs,
                                                             silu(__uint_as_float(v0[c + 2 * i + 1])) * __uint_as_float(v1[c + 2 * i + 1]) * rs);
                            *reinterpret_cast<uint4*>(dst + c) = pk;
                        }
                    }
                } else if (row_ok) {
                    __nv_bfloat16* dst = p.out + (size_t)row * p.ldc + hcol0 + pass * 64;
#pragma unroll
                    for (int part = 0; part < 2; ++part) {
#pragma unroll
                        for (int c = 0; c < 32; c += 8) {
                            uint4 pk;
                            __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const uint32_t lo = part ? v1[c + 2 * i] : v0[c + 2 * i];
                                const uint32_t hi = part ? v1[c + 2 * i + 1] : v0[c + 2 * i + 1];
                                q[i] = __floats2bfloat162_rn(__uint_as_float(lo) * rs, __uint_as_float(hi) * rs);
                            }
                            *reinterpret_cast<uint4*>(dst + part * 32 + c) = pk;
                        }
                    }
                }
            }
            if (quant) {
                // One scale per row and 128 output columns = the whole tile width: this thread holds
                // 64 of them, the warp with the other column half of the same rows the rest.  They
                // trade row maxima through shared memory, tagged with the tile number, in slots
                // that alternate from tile to tile.
                const unsigned seq = tile_no + 1u;
                volatile unsigned long long* slot_mine = &ctrl->amax_x[tile_no & 1u][half][r_in_tile];
                volatile unsigned long long* slot_other = &ctrl->amax_x[tile_no & 1u][half ^ 1][r_in_tile];
                *slot_mine = ((unsigned long long)seq << 32) | __float_as_uint(amax);
                unsigned long long other = 0;
                bool got = false;
                const long long t0 = clock64();
                for (unsigned i = 1;; ++i) {
                    other = *slot_other;
                    if ((unsigned)(other >> 32) == seq) {
                        got = true;
                        break;
                    }
                    if ((i & 255u) == 0 && (*failed || clock64() - t0 > p.budget)) break;
                }
                if (!__all_sync(ptx::kFullMask, got)) {
                    *failed = 1;
                    break;
                }
                float scale, inv;
                pow2_scale(fmaxf(amax, __uint_as_float((unsigned)(other & 0xffffffffull))), scale, inv);
                if (row_ok) {
                    unsigned char* dst = p.out_q + (size_t)row * p.ldc + hcol0 / 2;
#pragma unroll
                    for (int c = 0; c < 64; c += 16) {
                        uint4 pk;
                        unsigned short* q = reinterpret_cast<unsigned short*>(&pk);
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            q[i] = __nv_cvt_float2_to_fp8x2(make_float2(hval[c + 2 * i] * inv, hval[c + 2 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
                        *reinterpret_cast<uint4*>(dst + c) = pk;
                    }
                    if (half == 0) p.out_q_scale[(size_t)row * p.oqs0 + (size_t)(col0 / BN) * p.oqs1] = scale;
                }
            }
            ++acc_use;
        }
    }

    // ---- teardown -------------------------------------------------------------------------
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem, kTmemCols);
    }
    if (tid == 0) {
        if (ctrl->failed && p.error != nullptr) *p.error = 1;
        if (fused) {
            // the last CTA closes the receive side of the exchange
            __threadfence();
            if (atomicAdd(&fr.ws.ticket[0], 1u) == gridDim.x - 1) {
                fr.ws.ticket[0] = 0;
                fr.ws.epoch[0] = ep;
                __threadfence();
            }
        }
    }
}

constexpr int kSmemDense = kStages * kStageBytes + (int)((sizeof(Ctrl) + 15) & ~size_t(15)) + 1024;
constexpr int kSmemFused = kSmemDense + (int)sizeof(LayoutSmem);

template <bool kMx, bool kGather>
cudaError_t launch_one(const CUtensorMap& map_a, const CUtensorMap& map_w, const ExpertGemmArgs& args, const FusedReceive& fr, int ctas,
                       cudaStream_t stream) {
    const int smem = (kGather && fr.enabled) ? kSmemFused : kSmemDense;
    cudaError_t e = cudaFuncSetAttribute(expert_gemm_kernel<kMx, kGather>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemFused);
    if (e != cudaSuccess) return e;
    void* params[] = {const_cast<CUtensorMap*>(&map_a), const_cast<CUtensorMap*>(&map_w), const_cast<ExpertGemmArgs*>(&args),
                      const_cast<FusedReceive*>(&fr)};
    if (kGather && fr.enabled) {
        // every CTA's producer waits on rows that the index warps of all CTAs publish: the grid must be co-resident
        return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(expert_gemm_kernel<kMx, kGather>), dim3(ctas), dim3(kThreads), params,
                                           (size_t)smem, stream);
    }
    return cudaLaunchKernel(reinterpret_cast<const void*>(expert_gemm_kernel<kMx, kGather>), dim3(ctas), dim3(kThreads), params, (size_t)smem,
                            stream);
}

}  // namespace

int expert_gemm_smem_bytes(bool fused) { return fused ? kSmemFused : kSmemDense; }

cudaError_t launch_expert_gemm(const CUtensorMap& map_a, const CUtensorMap& map_w, const ExpertGemmArgs& args, bool gather,
                               const FusedReceive& fr, int ctas, cudaStream_t stream) {
    if (fr.enabled && !gather) return cudaErrorInvalidValue;
    if (args.mx) return gather ? launch_one<true, true>(map_a, map_w, args, fr, ctas, stream) : launch_one<true, false>(map_a, map_w, args, fr, ctas, stream);
    return gather ? launch_one<false, true>(map_a, map_w, args, fr, ctas, stream) : launch_one<false, false>(map_a, map_w, args, fr, ctas, stream);
}

}  // namespace afdep
