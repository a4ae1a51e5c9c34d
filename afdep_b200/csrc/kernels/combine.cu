// Attention-side combine: the return all-to-all and the top-k reduction in one kernel.
//
// One warp per token.  The warp already knows, from dispatch, which FFN ranks hold a reply
// row for the token and in which slot.  It polls the (local) per-slot reply flags those
// ranks release, then pulls every row with one non-multicast bulk load per FFN rank straight
// from that rank's heap over NVLink into shared memory, adds the rows in fp32 in rank order
// and writes the BF16 result in original token order.  No staging buffer on the attention
// rank and no separate gather or sum kernel, unlike the reference's pair of combine_impl and
// combine_reduce_epilogue_impl (deep_ep/include/deep_ep/impls/combine.cuh,
// combine_reduce_epilogue.cuh).
//
// Also here: the stand-alone barrier used by construction and close().
#include <cuda_bf16.h>

#include "afdep/kernels.h"
#include "afdep/status.cuh"

namespace afdep {

namespace {

constexpr int kBarBytes = 256;
constexpr int kMaxWarps = 16;

__global__ void __launch_bounds__(kMaxWarps * 32, 1)
collect_kernel(const RankCtx c, const AttnWs ws, unsigned char* __restrict__ out, int T) {
    extern __shared__ __align__(128) unsigned char smem[];
    const Geometry& g = c.g;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, NW = blockDim.x >> 5;
    const int G = gridDim.x, cta = blockIdx.x;
    const int F = g.ffn, C = g.capacity;
    const int ai = c.role_rank;
    const unsigned ep = ptx::ld_acquire_gpu(&ws.epoch[1]) + 1u;
    const WaitCtx wc{c.status, c.poison, c.budget, c.rank, /*kernel=*/5};
    unsigned char* heap = reinterpret_cast<unsigned char*>(c.peer[c.rank]);
    const uint32_t* reply_flag = reinterpret_cast<const uint32_t*>(heap + g.a_reply_flag);

    const int max_rows = F < g.top_k ? F : g.top_k;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    unsigned char* buf = smem + kBarBytes + (size_t)warp * max_rows * g.row_bytes;
    uint64_t* bar = &bars[warp];
    if (lane == 0) {
        ptx::mbar_init(bar, 1);
        ptx::fence_mbar_init();
    }
    __syncwarp();

    trace_stamp(c.trace, kTraceCollect, 0);
    const int nvec = g.hidden / 8;
    unsigned it = 0;
    for (int t = warp * G + cta; t < T; t += G * NW) {      // consecutive tokens on consecutive CTAs
        const int slot = (lane < F) ? ws.tok_slot[(size_t)t * F + lane] : -1;
        const unsigned mask = __ballot_sync(ptx::kFullMask, slot >= 0);
        unsigned char* dst = out + (size_t)t * g.row_bytes;
        if (mask == 0) {   // every choice of the token was -1 (or the token was rejected)
            for (int v = lane; v < nvec; v += 32) *reinterpret_cast<uint4*>(dst + (size_t)v * 16) = make_uint4(0, 0, 0, 0);
            continue;
        }
        bool ok = true;
        if (slot >= 0) {
            uint32_t seen = 0;
            ok = spin_until(wc, [&] {
                seen = ptx::ld_acquire_sys(reply_flag + (size_t)lane * C + slot);
                return seen == ep;
            });
            if (!ok) {
                report(wc, kTimeoutReply, lane, ep, ep, seen, t, slot);
                poison(wc);
            }
        }
        if (!__all_sync(ptx::kFullMask, ok)) break;
        if (it == 0) trace_stamp(c.trace, kTraceCollectFirst, 0);
        const int nrows = __popc(mask);
        if (lane == 0) {
            ptx::fence_proxy_async_global();
            ptx::mbar_expect_tx(bar, (uint32_t)nrows * g.row_bytes);
        }
        int r = 0;
        for (unsigned m = mask; m; m &= m - 1, ++r) {
            const int f = __ffs(m) - 1;
            const int s = __shfl_sync(ptx::kFullMask, slot, f);
            if (lane == 0)
                ptx::bulk_load(buf + (size_t)r * g.row_bytes,
                               c.peer[f] + g.f_reply + ((size_t)ai * C + s) * g.row_bytes, g.row_bytes, bar);
        }
        bool landed = spin_until(wc, [&] { return ptx::mbar_try_wait(bar, it & 1u); });
        if (!__all_sync(ptx::kFullMask, landed)) {
            if (lane == 0) {
                report(wc, kTimeoutReply, -1, ep, nrows, 0, t, -1);
                poison(wc);
            }
            break;
        }
        if (it == 0) trace_stamp(c.trace, kTraceCollectFirst, 1);
        ++it;
        if (nrows == 1) {
            for (int v = lane; v < nvec; v += 32)
                *reinterpret_cast<uint4*>(dst + (size_t)v * 16) = *reinterpret_cast<const uint4*>(buf + (size_t)v * 16);
        } else {
            for (int v = lane; v < nvec; v += 32) {
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (int rr = 0; rr < nrows; ++rr) {
                    const uint4 x = *reinterpret_cast<const uint4*>(buf + (size_t)rr * g.row_bytes + (size_t)v * 16);
                    const unsigned w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {     // BF16 -> fp32 is a shift / a mask; packed fp32 add
                        const float2 fl = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
                        const float2 r = __fadd2_rn(make_float2(acc[2 * i], acc[2 * i + 1]), fl);
                        acc[2 * i] = r.x;
                        acc[2 * i + 1] = r.y;
                    }
                }
                uint4 y;
                __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&y);
#pragma unroll
                for (int i = 0; i < 4; ++i) q[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
                *reinterpret_cast<uint4*>(dst + (size_t)v * 16) = y;
            }
        }
        __syncwarp();   // every lane is done with the buffer before the next bulk load lands
        if (it == 1) trace_stamp(c.trace, kTraceCollectFirst, 2);
    }

    __syncthreads();
    trace_stamp(c.trace, kTraceCollect, 2);
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(&ws.ticket[1], 1u) == (unsigned)(G - 1)) {
            ws.ticket[1] = 0;
            ws.epoch[1] = ep;
            __threadfence();
        }
    }
}

// Full barrier over all ranks of the Buffer: rank r writes the new epoch into word r of
// every peer's barrier array and waits until all words of its own array have reached it.
// Epochs only grow, so nothing is ever reset (the reference flips signs instead,
// deep_ep/include/deep_ep/common/comm.cuh:88-129).
__global__ void __launch_bounds__(32, 1) barrier_kernel(const RankCtx c, unsigned* epoch_word) {
    const int W = c.g.world;
    const int tid = threadIdx.x;
    const unsigned ep = *reinterpret_cast<volatile unsigned*>(epoch_word) + 1u;
    const WaitCtx wc{c.status, c.poison, c.budget, c.rank, /*kernel=*/6};
    if (tid < W) {
        __threadfence_system();
        ptx::st_release_sys(reinterpret_cast<uint32_t*>(c.peer[tid]) + c.rank, ep);
        const uint32_t* mine = reinterpret_cast<const uint32_t*>(c.peer[c.rank]) + tid;
        uint32_t seen = 0;
        const bool ok = spin_until(wc, [&] {
            seen = ptx::ld_acquire_sys(mine);
            return (int)(seen - ep) >= 0;
        });
        if (!ok) {
            report(wc, kTimeoutBarrier, tid, ep, ep, seen);
            poison(wc);
        }
    }
    __syncwarp();
    if (tid == 0) *epoch_word = ep;
}

}  // namespace

LaunchShape collect_shape(const Geometry& g, int tokens, int num_sms, int max_smem) {
    LaunchShape s{};
    const int max_rows = g.ffn < g.top_k ? g.ffn : g.top_k;
    int warps = (max_smem - kBarBytes) / (max_rows * g.row_bytes);
    if (warps > kMaxWarps) warps = kMaxWarps;
    if (warps < 1) warps = 1;
    // Few tokens: one per CTA rather than a full CTA of warps on a few SMs, so that every
    // token's rows come in through a different SM's copy engine.
    int ctas = num_sms;
    int want = tokens < 1 ? 1 : tokens;
    if (ctas > want) ctas = want;
    s.ctas = ctas;
    s.warps = warps;
    s.smem_bytes = kBarBytes + warps * max_rows * g.row_bytes;
    return s;
}

cudaError_t launch_collect(const RankCtx& c, const AttnWs& ws, void* out, int T, LaunchShape s,
                           cudaStream_t stream) {
    collect_kernel<<<s.ctas, s.warps * 32, s.smem_bytes, stream>>>(c, ws, static_cast<unsigned char*>(out), T);
    return cudaGetLastError();
}

cudaError_t launch_barrier(const RankCtx& c, unsigned* epoch_word, cudaStream_t stream) {
    barrier_kernel<<<1, 32, 0, stream>>>(c, epoch_word);
    return cudaGetLastError();
}

cudaError_t configure_dispatch(int max_smem);
cudaError_t configure_ffn(int max_smem);

cudaError_t configure_kernels(int max_smem) {
    cudaError_t e = configure_dispatch(max_smem);
    if (e != cudaSuccess) return e;
    e = configure_ffn(max_smem);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(collect_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
}

}  // namespace afdep
