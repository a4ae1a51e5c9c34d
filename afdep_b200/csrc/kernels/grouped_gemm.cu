// Grouped expert GEMM on tcgen05: C[rows, N] = A[rows, K] * W_e[N, K]^T for the expert-major
// rows that worker_receive returns, one weight matrix per local expert.
//
// Layout of a CTA (persistent over 128 x 256 output tiles):
//   warp 0      TMA producer: tensor-map loads of a 128 x BK tile of A and a 256 x BK tile of
//               the expert's W into a ring of 128-byte-swizzled shared-memory stages
//   warp 1      allocates tensor memory, then one elected lane issues tcgen05.mma (M 128, N 256)
//               for every stage and commits stage-free / accumulator-ready mbarriers
//   epilogue    warps 2..: tcgen05.ld the fp32 accumulator (thread = tile row, one column part
//               per warp), apply the block scales (FP8), SwiGLU and the routing weight, store
//               BF16.  BF16 uses sixteen warps of 64 columns; FP8 keeps 128 running sums per
//               thread for the promotion and uses eight warps of 128 columns (measured: sixteen
//               warps cap the kernel at 96 registers and spill the sums).
// Two 256-column accumulators fill tensor memory and let the MMAs of the next tile (BF16) or
// the next K block (FP8) run while the epilogue warps drain the previous one.
//
// BF16 mode: kind::f16, BK = 64, one commit per tile.
// FP8 mode:  kind::f8f6f4 on e4m3 with fp32 scales: one scale per row and 128 columns of A,
//            one per 128 x 128 block of W.  Every 128-deep K block is multiplied into a fresh
//            TMEM accumulator and promoted by the epilogue warps: acc += tmem * a_s * w_s.
// SwiGLU:    gate and up rows of W alternate in blocks of 32, so every 64-column part of a tile
//            holds 32 gate columns followed by their 32 up columns; the output has N/2 columns.
//
// Expert segments start on multiples of `alignment` rows (a multiple of 128), so a 128-row
// tile never straddles two experts; tiles past an expert's last row are skipped, rows past it
// inside the last tile are padding.  The reference library has no GEMM at all (callers bring
// their own); this kernel is the expert path of the end-to-end benchmark.
#include <mutex>

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "afdep/gemm_api.h"
#include "afdep/tcgen05.cuh"

namespace afdep {

namespace {

constexpr int BM = 128, BN = 256;
// columns one epilogue warp handles / epilogue warps / threads, per operand type
__host__ __device__ constexpr int part_cols(bool fp8) { return fp8 ? 128 : 64; }
__host__ __device__ constexpr int epi_warps(bool fp8) { return 4 * (BN / part_cols(fp8)); }      // four lane quarters times the column parts
__host__ __device__ constexpr int cta_threads(bool fp8) { return (2 + epi_warps(fp8)) * 32; }
constexpr int kStageBytes = (BM + BN) * 128;  // A tile + W tile, 128-byte rows
constexpr int kStages = 4;
constexpr int kTmemCols = 512;                // two 256-column fp32 accumulators
constexpr unsigned kSpinLimit = 1u << 28;     // try_wait probes before a wait gives up

struct Ctrl {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int failed;
    int tile_prefix[kMaxExpertsLocal + 1];    // tiles of experts [0, e), in units of (m tiles * n tiles)
    int seg_start[kMaxExpertsLocal];
    // FP8 output: (tile number << 32 | row amax bits) per [tile parity][column half][tile row], so
    // the two warps that hold the halves of a 128-column scale group can agree on its scale
    unsigned long long amax_x[2][2][BM];
};

// Bounded mbarrier wait: gives up (and makes every role leave) instead of hanging.
__device__ __forceinline__ bool wait_bar(uint64_t* bar, unsigned parity, volatile int* failed) {
    for (unsigned i = 0; i < kSpinLimit; ++i) {
        if (ptx::mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *failed) return false;
    }
    *failed = 1;
    return false;
}

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

template <bool kFp8>
__global__ void __launch_bounds__(cta_threads(kFp8), 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const GroupedGemmArgs p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // 1024-byte alignment for the swizzled stages, whatever the base of dynamic shared memory is
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem + kStages * kStageBytes);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int BK = kFp8 ? 128 : 64;          // elements per 128-byte row
    constexpr int HN = part_cols(kFp8);
    constexpr int kEpiWarps = epi_warps(kFp8);
    const int num_kb = p.K / BK;
    const int n_tiles = (p.N + BN - 1) / BN;     // the last tile may be half empty (N a multiple of 128)

    // ---- set-up: barriers, tile schedule, tensor memory --------------------------------
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(&ctrl->full[s], 1);
            ptx::mbar_init(&ctrl->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(&ctrl->acc_full[b], 1);
            ptx::mbar_init(&ctrl->acc_empty[b], kEpiWarps);     // one arrival per epilogue warp
        }
        ctrl->failed = 0;
        ptx::fence_mbar_init();
        // experts -> tiles: expert e owns rows [seg_start[e], ends[e]), seg_start aligned
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
        tc::prefetch_tensormap(&map_a);
        tc::prefetch_tensormap(&map_w);
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = ctrl->tmem_base;
    const int total_work = ctrl->tile_prefix[p.experts];
    volatile int* failed = &ctrl->failed;

    // Work item -> (expert, first row, first column).  Within an expert, row tiles vary fastest
    // so that CTAs working side by side share the expert's weight tile in L2.
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
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            unsigned phase = 0;
            for (int w = blockIdx.x; w < total_work; w += gridDim.x) {
                int e, row0, col0;
                decode(w, e, row0, col0);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!wait_bar(&ctrl->empty[stage], phase ^ 1u, failed)) break;
                    unsigned char* sa = smem + stage * kStageBytes;
                    ptx::mbar_expect_tx(&ctrl->full[stage], kStageBytes);
                    tc::tma_load_2d(sa, &map_a, kb * BK, row0, &ctrl->full[stage]);
                    tc::tma_load_2d(sa + BM * 128, &map_w, kb * BK, e * p.N + col0, &ctrl->full[stage]);
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
            constexpr uint32_t idesc = tc::instr_desc(BM, BN, kFp8 ? 0u : 1u, kFp8 ? 0u : 1u);
            constexpr int kMmaK = 32;            // bytes of K one instruction consumes
            int stage = 0;
            unsigned phase = 0;
            int acc_use = 0;                     // accumulator buffers handed out so far
            for (int w = blockIdx.x; w < total_work && !*failed; w += gridDim.x) {
                for (int kb = 0; kb < num_kb; ++kb) {
                    const bool new_acc = kFp8 || kb == 0;
                    const int buf = acc_use & 1;
                    if (new_acc) {
                        // the epilogue must have drained this accumulator's previous contents
                        if (!wait_bar(&ctrl->acc_empty[buf], ((acc_use >> 1) & 1u) ^ 1u, failed)) break;
                        tc::fence_after_sync();
                    }
                    if (!wait_bar(&ctrl->full[stage], phase, failed)) break;
                    tc::fence_after_sync();
                    const unsigned char* sa = smem + stage * kStageBytes;
                    const unsigned char* sb = sa + BM * 128;
                    const uint32_t d = tmem + (uint32_t)buf * BN;
#pragma unroll
                    for (int k = 0; k < 128 / kMmaK; ++k) {
                        const uint64_t da = tc::smem_desc_sw128(sa + k * kMmaK);
                        const uint64_t db = tc::smem_desc_sw128(sb + k * kMmaK);
                        const bool acc = kFp8 ? (k > 0) : (kb > 0 || k > 0);
                        if (kFp8)
                            tc::mma_fp8(d, da, db, idesc, acc);
                        else
                            tc::mma_bf16(d, da, db, idesc, acc);
                    }
                    tc::mma_commit(&ctrl->empty[stage]);          // stage reusable once these MMAs are done
                    if (kFp8 || kb == num_kb - 1) {
                        tc::mma_commit(&ctrl->acc_full[buf]);     // accumulator ready for the epilogue
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
        const int quarter = warp & 3;            // TMEM lanes this warp may touch: [32 * quarter, +32)
        const int half = (warp - 2) >> 2;        // which HN columns of the tile this warp handles
        const int r_in_tile = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        int acc_use = 0;
        unsigned tile_no = 0;                    // tiles this CTA has finished, the same in every warp
        for (int w = blockIdx.x; w < total_work && !*failed; w += gridDim.x, ++tile_no) {
            int e, row0, col0;
            decode(w, e, row0, col0);
            const int hcol0 = col0 + half * HN;                 // first column of this warp's half
            const bool half_ok = hcol0 < p.N;
            const int row = row0 + r_in_tile;
            const bool row_ok = row < p.ends[e] && row < p.rows && half_ok;
            float acc[kFp8 ? HN : 1];
            if (kFp8) {
#pragma unroll
                for (int c = 0; c < HN; ++c) acc[kFp8 ? c : 0] = 0.f;
            }
            bool ok = true;
            if (kFp8) {
                // promotion: one fresh accumulator per 128-deep K block
                const float* a_sc = p.a_scale + (size_t)(row_ok ? row : 0) * p.a_scale_s0;
                const float* w_sc = p.w_scale + ((size_t)e * (p.N / 128) + (half_ok ? hcol0 / 128 : 0)) * (p.K / 128);
                float s_next = a_sc[0] * w_sc[0];
                for (int kb = 0; kb < num_kb; ++kb) {
                    const int buf = acc_use & 1;
                    const float s = s_next;
                    if (kb + 1 < num_kb) s_next = a_sc[(size_t)(kb + 1) * p.a_scale_s1] * w_sc[kb + 1];
                    if (!wait_bar(&ctrl->acc_full[buf], (acc_use >> 1) & 1u, failed)) {
                        ok = false;
                        break;
                    }
                    tc::fence_after_sync();
                    // Two register tiles in ping-pong: the tcgen05.ld of the next 32 columns is in
                    // flight while the packed FMAs of the current 32 run (two fp32 lanes per
                    // instruction on sm_100), so the promotion stays shorter than the MMAs it hides behind.
                    const float2 s2 = make_float2(s, s);
                    const uint32_t tsrc = tmem + lane_base + (uint32_t)(buf * BN + half * HN);
                    uint32_t va[32], vb[32];
                    auto promote = [&](const uint32_t (&v)[32], int ch) {
#pragma unroll
                        for (int c = 0; c < 32; c += 2) {
                            const int i0 = kFp8 ? ch * 32 + c : 0;
                            const float2 r = __ffma2_rn(make_float2(__uint_as_float(v[c]), __uint_as_float(v[c + 1])), s2,
                                                        make_float2(acc[i0], acc[kFp8 ? i0 + 1 : 0]));
                            acc[i0] = r.x;
                            acc[kFp8 ? i0 + 1 : 0] = r.y;
                        }
                    };
                    tc::tmem_ld32(tsrc, va);
                    tc::tmem_ld_wait_on(va);
#pragma unroll
                    for (int ch = 0; ch < HN / 32; ch += 2) {
                        tc::tmem_ld32(tsrc + (uint32_t)((ch + 1) * 32), vb);
                        promote(va, ch);
                        tc::tmem_ld_wait_on(vb);
                        if (ch + 2 < HN / 32) tc::tmem_ld32(tsrc + (uint32_t)((ch + 2) * 32), va);
                        promote(vb, ch + 1);
                        if (ch + 2 < HN / 32) tc::tmem_ld_wait_on(va);
                    }
                    tc::fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&ctrl->acc_empty[buf]);
                    ++acc_use;
                }
                if (!ok) break;
            }
            int buf = 0;
            if (!kFp8) {
                buf = acc_use & 1;
                if (!wait_bar(&ctrl->acc_full[buf], (acc_use >> 1) & 1u, failed)) break;
                tc::fence_after_sync();
            }
            // ---- write the half tile: thread = one row, 32 columns at a time -----------------
            const float rs = (p.row_scale != nullptr && row_ok) ? p.row_scale[row] : 1.f;
            __nv_bfloat16* out_row = p.out + (size_t)(row_ok ? row : 0) * p.ldc;
            const uint32_t tbase = tmem + lane_base + (uint32_t)(buf * BN + half * HN);
            if (kFp8 && p.swiglu && p.out_q != nullptr) {
                // SwiGLU output quantised to e4m3 in the epilogue.  This thread holds 64 of the 128
                // output columns of its row's scale group (the tile's 256 gate|up columns); the
                // warp with the other column half of the same rows holds the rest.  The two trade
                // their row maxima through shared memory, tagged with the tile number, in a slot
                // pair that alternates from tile to tile (a warp cannot run two tiles ahead of its
                // partner, because it needs the partner's value for the tile in between).
                float m = 0.f;
#pragma unroll
                for (int sub = 0; sub < HN / 64; ++sub) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const int ig = kFp8 ? sub * 64 + c : 0, iu = kFp8 ? sub * 64 + 32 + c : 0;
                        const float hval = silu(acc[ig]) * acc[iu] * rs;
                        acc[ig] = hval;          // the gate slot now holds the output value
                        m = fmaxf(m, fabsf(hval));
                    }
                }
                const unsigned seq = tile_no + 1u;
                volatile unsigned long long* slot_mine = &ctrl->amax_x[tile_no & 1u][half][r_in_tile];
                volatile unsigned long long* slot_other = &ctrl->amax_x[tile_no & 1u][half ^ 1][r_in_tile];
                *slot_mine = ((unsigned long long)seq << 32) | __float_as_uint(m);
                unsigned long long other = 0;
                bool got = false;
                for (unsigned i = 0; i < kSpinLimit; ++i) {
                    other = *slot_other;
                    if ((unsigned)(other >> 32) == seq) {
                        got = true;
                        break;
                    }
                    if ((i & 1023u) == 1023u && *failed) break;
                }
                if (!got) {
                    *failed = 1;
                    break;
                }
                m = fmaxf(fmaxf(m, __uint_as_float((unsigned)(other & 0xffffffffull))), 1e-12f);
                const float inv = 448.f / m;
                if (row_ok) {
                    unsigned char* dst = p.out_q + (size_t)row * p.ldc + hcol0 / 2;
#pragma unroll
                    for (int sub = 0; sub < HN / 64; ++sub) {
#pragma unroll
                        for (int c = 0; c < 32; c += 16) {
                            uint4 pk;
                            unsigned short* q = reinterpret_cast<unsigned short*>(&pk);
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const int i0 = kFp8 ? sub * 64 + c + 2 * i : 0;
                                q[i] = __nv_cvt_float2_to_fp8x2(make_float2(acc[i0] * inv, acc[kFp8 ? i0 + 1 : 0] * inv), __NV_SATFINITE, __NV_E4M3);
                            }
                            *reinterpret_cast<uint4*>(dst + sub * 32 + c) = pk;
                        }
                    }
                    if (half == 0) p.out_q_scale[(size_t)row * p.oqs0 + (size_t)(col0 / BN) * p.oqs1] = m / 448.f;
                }
            } else if (p.swiglu) {
                // every 64 columns hold 32 gate columns followed by their 32 up columns
#pragma unroll
                for (int sub = 0; sub < HN / 64; ++sub) {
                    float gt[32], up[32];
                    if (kFp8) {
#pragma unroll
                        for (int c = 0; c < 32; ++c) {
                            gt[c] = acc[kFp8 ? sub * 64 + c : 0];
                            up[c] = acc[kFp8 ? sub * 64 + 32 + c : 0];
                        }
                    } else {
                        uint32_t v0[32], v1[32];
                        tc::tmem_ld32(tbase + (uint32_t)(sub * 64), v0);
                        tc::tmem_ld32(tbase + (uint32_t)(sub * 64 + 32), v1);
                        tc::tmem_ld_wait_on(v0);
                        tc::tmem_ld_wait_on(v1);
#pragma unroll
                        for (int c = 0; c < 32; ++c) {
                            gt[c] = __uint_as_float(v0[c]);
                            up[c] = __uint_as_float(v1[c]);
                        }
                    }
                    if (row_ok) {
                        __nv_bfloat16* dst = out_row + hcol0 / 2 + sub * 32;
#pragma unroll
                        for (int c = 0; c < 32; c += 8) {
                            uint4 pk;
                            __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                q[i] = __floats2bfloat162_rn(silu(gt[c + 2 * i]) * up[c + 2 * i] * rs,
                                                             silu(gt[c + 2 * i + 1]) * up[c + 2 * i + 1] * rs);
                            *reinterpret_cast<uint4*>(dst + c) = pk;
                        }
                    }
                }
            } else {
#pragma unroll
                for (int ch = 0; ch < HN / 32; ++ch) {
                    float val[32];
                    if (kFp8) {
#pragma unroll
                        for (int c = 0; c < 32; ++c) val[c] = acc[kFp8 ? ch * 32 + c : 0];
                    } else {
                        uint32_t v[32];
                        tc::tmem_ld32(tbase + (uint32_t)(ch * 32), v);
                        tc::tmem_ld_wait_on(v);
#pragma unroll
                        for (int c = 0; c < 32; ++c) val[c] = __uint_as_float(v[c]);
                    }
                    if (row_ok) {
                        __nv_bfloat16* dst = out_row + hcol0 + ch * 32;
#pragma unroll
                        for (int c = 0; c < 32; c += 8) {
                            uint4 pk;
                            __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                q[i] = __floats2bfloat162_rn(val[c + 2 * i] * rs, val[c + 2 * i + 1] * rs);
                            *reinterpret_cast<uint4*>(dst + c) = pk;
                        }
                    }
                }
            }
            if (!kFp8) {
                tc::fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&ctrl->acc_empty[buf]);
                ++acc_use;
            }
        }
    }

    // ---- teardown: everybody is done with tensor memory before it is released ------------
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

int grouped_gemm_smem_bytes() { return kSmemBytes; }

GemmErrorWord gemm_error_word(int device_ordinal) {
    static std::mutex mu;
    static GemmErrorWord words[64] = {};
    std::lock_guard<std::mutex> lock(mu);
    if (device_ordinal < 0 || device_ordinal >= 64) return GemmErrorWord{nullptr, nullptr};
    GemmErrorWord& w = words[device_ordinal];
    if (w.host == nullptr) {
        void* host = nullptr;
        void* dev = nullptr;
        if (cudaHostAlloc(&host, 64, cudaHostAllocMapped) != cudaSuccess) return GemmErrorWord{nullptr, nullptr};
        *static_cast<int*>(host) = 0;
        if (cudaHostGetDevicePointer(&dev, host, 0) != cudaSuccess) {
            cudaFreeHost(host);
            return GemmErrorWord{nullptr, nullptr};
        }
        w.host = static_cast<volatile int*>(host);
        w.device = static_cast<int*>(dev);
    }
    return w;
}

cudaError_t launch_grouped_gemm(const CUtensorMap& map_a, const CUtensorMap& map_w, const GroupedGemmArgs& args, int ctas,
                                cudaStream_t stream) {
    // The attribute belongs to the current device's context, so it is set on every launch
    // (a cheap call) rather than remembered per process.
    cudaError_t e = args.fp8 ? cudaFuncSetAttribute(grouped_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes)
                             : cudaFuncSetAttribute(grouped_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    if (args.fp8)
        grouped_gemm_kernel<true><<<ctas, cta_threads(true), kSmemBytes, stream>>>(map_a, map_w, args);
    else
        grouped_gemm_kernel<false><<<ctas, cta_threads(false), kSmemBytes, stream>>>(map_a, map_w, args);
    return cudaGetLastError();
}

}  // namespace afdep
