// Attention-side dispatch: route guard, deterministic layout and payload push in ONE launch.
//
// Phase 1 (layout) — every CTA owns a contiguous chunk of tokens.  Its warps rank each
// (token, k) choice among the earlier choices of the same expert and each (token, FFN rank)
// record among the earlier records for that rank, first inside the warp's sub-range, then
// across warps (shared-memory scan), then across CTAs (decoupled look-back over epoch-tagged
// aggregates in global memory).  The result is a placement that depends only on the inputs:
// record slot = number of earlier tokens of this source that also go to that FFN rank, and
// pos = number of earlier choices of that expert by this source.  The last CTA ends up with
// the source's totals and pushes them to the FFN ranks (the count "all-to-all") before any
// payload leaves.
//
// Phase 2 (push) — one warp per token: a bulk async copy brings the row into shared memory
// once, lanes append scales/routes/weights, and one bulk store per destination FFN rank
// writes the finished record straight into that rank's staging slot over NVLink.  Once a
// store group has completed, the data warp hands the token to the CTA's flag warp, which
// issues the system-scope fence and the 4-byte arrival flag per record; the receiver can
// start on a record as soon as it has landed, and the (slow) fence never stalls a data warp.
//
// Replaces, for the AFD case, the reference's dispatch_impl (notify + dispatch warps,
// deep_ep/include/deep_ep/impls/dispatch.cuh:18-433), its deterministic prologue
// (dispatch_deterministic_prologue.cuh) and the stand-alone route guard (afdep_roles.cuh:11-33)
// without the two grid-wide GPU barriers those need, and never traps on a bad route.
#include "afdep/kernels.h"
#include "afdep/route_layout.cuh"
#include "afdep/status.cuh"

namespace afdep {

namespace {

constexpr int kBarBytes = 1024;   // mbarrier area at the start of dynamic shared memory
constexpr int kMaxWarps = 16;
constexpr int kMaxCtas = 160;

// NB record buffers per warp form a ring: while token i is being stored, token i+1 is
// already loading, and the arrival flags of token i-(NB-2) are released once its store group
// has completed.  NB = 2 degenerates to load -> store -> wait -> flag.
template <int NB>
__global__ void __launch_bounds__(kMaxWarps * 32, 1)
dispatch_kernel(const RankCtx c, const AttnWs ws, const DispatchArgs a) {
    constexpr int L = NB - 2;     // how many tokens the flag release lags behind the stores
    extern __shared__ __align__(128) unsigned char smem[];
    const Geometry& g = c.g;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, NW = blockDim.x >> 5;
    const int G = gridDim.x, cta = blockIdx.x;
    const int F = g.ffn, K = g.top_k, E = g.num_experts, EL = g.experts_local, C = g.capacity;
    const int ai = c.role_rank;
    const unsigned ep = ptx::ld_acquire_gpu(&ws.epoch[0]) + 1u;
    const WaitCtx wc{c.status, c.poison, c.budget, c.rank, /*kernel=*/1};
    (void)L;
    trace_stamp(c.trace, kTraceDispatch, 0);

    const int T = a.T;
    const int chunk = (T + G - 1) / G;
    const int t0 = min(T, cta * chunk), t1 = min(T, t0 + chunk);

    // ------------------------------------------------------------------ phase 1: layout
    int *tot = nullptr, *lb = nullptr;
    const RouteLayoutOut lo{ws.route_e, ws.route_pos, ws.tok_slot};
    bool alive = route_layout_phase(a.ids, T, K, E, EL, F, ep, ws.agg, lo, reinterpret_cast<int*>(smem + kBarBytes), wc,
                                    &tot, &lb);

    // The last CTA now holds this source's totals: push them to the FFN ranks.
    if (cta == G - 1 && alive) {
        const int cs = cnt_stride(g);
        for (int idx = tid; idx < F * (EL + 1); idx += blockDim.x) {
            const int f = idx / (EL + 1), el = idx - f * (EL + 1);
            const int col = (el < EL) ? (F + f * EL + el) : f;
            int* dst = reinterpret_cast<int*>(c.peer[f] + g.f_cnt) + (size_t)ai * cs + el;
            *reinterpret_cast<volatile int*>(dst) = lb[col] + tot[col];
        }
        __syncthreads();
        if (tid < F) {
            ptx::fence_acq_rel_sys();
            ptx::st_relaxed_sys(reinterpret_cast<uint32_t*>(c.peer[tid] + g.f_cnt_flag) + ai * 32, ep);
        }
    }
    // Shared memory changes hands from generic-proxy scratch to bulk-copy buffers.
    ptx::fence_proxy_async_smem();
    __syncthreads();
    trace_stamp(c.trace, kTraceDispatch, 1);

    // ------------------------------------------------------------------ phase 2: push
    // Warps [0, ND) move data; the last warp releases arrival flags.
    const int ND = NW - 1;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    int* done_cnt = reinterpret_cast<int*>(smem + kBarBytes - 128);   // [ND] tokens completed per data warp
    unsigned char* bufs = smem + kBarBytes + (size_t)warp * NB * g.rec_bytes;
    if (warp < ND && lane == 0) {
        for (int b = 0; b < NB; ++b) ptx::mbar_init(&bars[warp * NB + b], 1);
        ptx::fence_mbar_init();
    }
    if (tid < 32) done_cnt[tid] = 0;
    __syncthreads();

    const unsigned char* xb = static_cast<const unsigned char*>(a.x);
    const int sg = g.fp8 ? g.scale_groups : 0;
    auto tokens_of = [&](int w) { return (alive && t0 + w < t1) ? (t1 - (t0 + w) + ND - 1) / ND : 0; };

    if (warp < ND) {
        const int first = t0 + warp;
        const int n_w = tokens_of(warp);
        unsigned phase_bits = 0;      // lane 0: parity of each buffer's mbarrier

        // A(i): start loading token i into its ring buffer and append its metadata.
        auto stage = [&](int i, int& slot, unsigned& mask) {
            const int t = first + i * ND;
            slot = (lane < F) ? ws.tok_slot[(size_t)t * F + lane] : -1;
            mask = __ballot_sync(ptx::kFullMask, slot >= 0);
            if (mask == 0) return;
            unsigned char* buf = bufs + (size_t)(i % NB) * g.rec_bytes;
            if (lane == 0) {
                uint64_t* bar = &bars[warp * NB + (i % NB)];
                ptx::mbar_expect_tx(bar, g.payload_bytes);
                ptx::bulk_load(buf, xb + (size_t)t * g.payload_bytes, g.payload_bytes, bar);
            }
            int* meta = reinterpret_cast<int*>(buf + g.meta_off);
            if (lane < K) {
                meta[lane] = ws.route_e[(size_t)t * K + lane];
                meta[K + lane] = ws.route_pos[(size_t)t * K + lane];
                reinterpret_cast<float*>(meta)[2 * K + lane] = a.weights[(size_t)t * K + lane];
            }
            if (lane == 0) meta[3 * K] = t;
            for (int gi = lane; gi < sg; gi += 32)
                reinterpret_cast<float*>(buf + g.payload_bytes)[gi] = a.x_scale[(size_t)t * a.ss0 + (size_t)gi * a.ss1];
            ptx::fence_proxy_async_smem();
        };

        int slot_c = -1, slot_n = -1;
        unsigned mask_c = 0, mask_n = 0;
        bool ok = true;
        if (n_w > 0) stage(0, slot_c, mask_c);
        for (int i = 0; i < n_w; ++i) {
            // Buffer (i+1) % NB last held token i+1-NB, whose stores completed at step i-1.
            if (i + 1 < n_w) stage(i + 1, slot_n, mask_n);
            __syncwarp();
            if (mask_c) {
                const int b = i % NB;
                unsigned char* buf = bufs + (size_t)b * g.rec_bytes;
                if (lane == 0) {
                    uint64_t* bar = &bars[warp * NB + b];
                    const unsigned parity = (phase_bits >> b) & 1u;
                    // A local bulk load always completes; the bound only guards against a broken build.
                    ok = spin_until(wc, [&] { return ptx::mbar_try_wait(bar, parity); });
                    phase_bits ^= 1u << b;
                }
                ok = __shfl_sync(ptx::kFullMask, ok, 0);
                if (!ok) break;
                const int t = first + i * ND;
                for (unsigned m = mask_c; m; m &= m - 1) {
                    const int f = __ffs(m) - 1;
                    const int s = __shfl_sync(ptx::kFullMask, slot_c, f);
                    if (lane == 0) {
                        const bool inb = !c.bounds_check || (s >= 0 && s < C);
                        if (inb)
                            ptx::bulk_store(c.peer[f] + g.f_stage + ((size_t)ai * C + s) * g.rec_bytes, buf, g.rec_bytes);
                        else
                            report(wc, kBadIndex, f, ep, C, s, t, 1);
                    }
                }
            }
            if (lane == 0) {
                ptx::bulk_commit();            // one group per token, possibly empty
                if (i >= L) {
                    ptx::bulk_wait<L>();       // token i-L has fully landed at its destinations
                    ptx::st_release_cta_shared(&done_cnt[warp], i - L + 1);
                }
            }
            slot_c = slot_n;
            mask_c = mask_n;
        }
        if (lane == 0) {
            ptx::bulk_wait<0>();
            ptx::st_release_cta_shared(&done_cnt[warp], ok ? n_w : -1);
        }
    } else {
        // Flag warp: lane w follows data warp w.
        const int mine = (lane < ND) ? tokens_of(lane) : 0;
        int flagged = 0;
        bool aborted = false;
        const long long t_begin = clock64();
        unsigned idle = 0;
        while (true) {
            int d = (lane < ND && !aborted) ? ptx::ld_acquire_cta_shared(&done_cnt[lane]) : flagged;
            if (d < 0) {
                aborted = true;
                d = flagged;
            }
            if (d > flagged) {
                ptx::fence_acq_rel_sys();
                for (int j = flagged; j < d; ++j) {
                    const int t = t0 + lane + j * ND;
                    for (int f = 0; f < F; ++f) {
                        const int s = ws.tok_slot[(size_t)t * F + f];
                        if (s >= 0 && s < C)
                            ptx::st_relaxed_sys(reinterpret_cast<uint32_t*>(c.peer[f] + g.f_slot_flag) + (size_t)ai * C + s, ep);
                    }
                }
                flagged = d;
                idle = 0;
            }
            const bool fin = lane >= ND || aborted || flagged >= mine;
            if (__all_sync(ptx::kFullMask, fin)) break;
            if (++idle > 1) __nanosleep(64);
            if ((idle & 255u) == 0 && (poisoned(wc) || clock64() - t_begin > 4 * c.budget)) break;
        }
    }

    // The last CTA to get here closes the exchange on this side.
    __syncthreads();
    trace_stamp(c.trace, kTraceDispatch, 2);
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(&ws.ticket[0], 1u) == (unsigned)(G - 1)) {
            ws.ticket[0] = 0;
            ws.epoch[0] = ep;
            __threadfence();
        }
    }
}

// Opt-in shared memory left for the dynamic part, set by configure_dispatch.
int g_dyn_smem = 227 * 1024 - 256;

int pick_buffers(const Geometry& g) {
    // Deepest ring that still leaves enough warps per CTA to hide the layout phase.
    const int avail = g_dyn_smem - kBarBytes;
    if (avail / (4 * g.rec_bytes) >= 6) return 4;
    if (avail / (3 * g.rec_bytes) >= 3) return 3;
    return 2;
}

}  // namespace

int max_dispatch_ctas() { return kMaxCtas; }

LaunchShape dispatch_shape(const Geometry& g, int tokens, int num_sms, int max_smem) {
    LaunchShape s{};
    const int ncols = g.ffn + g.num_experts;
    (void)max_smem;
    const int max_dyn = g_dyn_smem;
    const int nb = pick_buffers(g);
    int data_warps = (max_dyn - kBarBytes) / (nb * g.rec_bytes);
    if (data_warps > kMaxWarps - 1) data_warps = kMaxWarps - 1;
    if (data_warps < 1) data_warps = 1;
    int warps = data_warps + 1;          // plus the flag warp
    // Phase 1 scratch must fit too.
    while (warps > 2 && kBarBytes + route_layout_scratch_ints(warps, ncols) * 4 > max_dyn) --warps;
    int ctas = num_sms < kMaxCtas ? num_sms : kMaxCtas;
    // No point in more CTAs than there are warp-sized groups of tokens.
    int want = (tokens + warps - 2) / (warps - 1);
    if (want < 1) want = 1;
    if (ctas > want) ctas = want;
    if (ctas < 1) ctas = 1;
    s.ctas = ctas;
    s.warps = warps;
    const int p1 = kBarBytes + route_layout_scratch_ints(warps, ncols) * 4;
    const int p2 = kBarBytes + (warps - 1) * nb * g.rec_bytes;
    s.smem_bytes = p1 > p2 ? p1 : p2;
    return s;
}

cudaError_t launch_dispatch(const RankCtx& c, const AttnWs& ws, const DispatchArgs& a, LaunchShape s,
                            cudaStream_t stream) {
    switch (pick_buffers(c.g)) {
        case 4: dispatch_kernel<4><<<s.ctas, s.warps * 32, s.smem_bytes, stream>>>(c, ws, a); break;
        case 3: dispatch_kernel<3><<<s.ctas, s.warps * 32, s.smem_bytes, stream>>>(c, ws, a); break;
        default: dispatch_kernel<2><<<s.ctas, s.warps * 32, s.smem_bytes, stream>>>(c, ws, a); break;
    }
    return cudaGetLastError();
}

cudaError_t configure_dispatch(int max_smem) {
    cudaFuncAttributes attr;
    cudaError_t e = cudaFuncGetAttributes(&attr, dispatch_kernel<4>);
    if (e != cudaSuccess) return e;
    g_dyn_smem = max_smem - (int)attr.sharedSizeBytes - 128;
    e = cudaFuncSetAttribute(dispatch_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, g_dyn_smem);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(dispatch_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, g_dyn_smem);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(dispatch_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, g_dyn_smem);
}

}  // namespace afdep
