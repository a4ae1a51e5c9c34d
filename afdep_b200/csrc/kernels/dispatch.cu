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
// writes the finished record straight into that rank's staging slot over NVLink.  After a
// store group has completed, the warp releases one 4-byte arrival flag per record, so the
// receiver can start on a record as soon as it has landed.
//
// Replaces, for the AFD case, the reference's dispatch_impl (notify + dispatch warps,
// deep_ep/include/deep_ep/impls/dispatch.cuh:18-433), its deterministic prologue
// (dispatch_deterministic_prologue.cuh) and the stand-alone route guard (afdep_roles.cuh:11-33)
// without the two grid-wide GPU barriers those need, and never traps on a bad route.
#include "afdep/kernels.h"
#include "afdep/status.cuh"

namespace afdep {

namespace {

constexpr int kNB = 2;            // record buffers per warp
constexpr int kBarBytes = 1024;   // mbarrier area at the start of dynamic shared memory
constexpr int kMaxWarps = 16;
constexpr int kMaxCtas = 160;

__device__ __forceinline__ int align_up_dev(int v, int a) { return (v + a - 1) / a * a; }

__global__ void __launch_bounds__(kMaxWarps * 32, 1)
dispatch_kernel(const RankCtx c, const AttnWs ws, const DispatchArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    const Geometry& g = c.g;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, NW = blockDim.x >> 5;
    const int G = gridDim.x, cta = blockIdx.x;
    const int F = g.ffn, K = g.top_k, E = g.num_experts, EL = g.experts_local, C = g.capacity;
    const int ncols = F + E;
    const int ai = c.role_rank;
    const unsigned ep = ptx::ld_acquire_gpu(&ws.epoch[0]) + 1u;
    const WaitCtx wc{c.status, c.poison, c.budget, c.rank, /*kernel=*/1};

    const int T = a.T;
    const int chunk = (T + G - 1) / G;
    const int t0 = min(T, cta * chunk), t1 = min(T, t0 + chunk);
    const int n = t1 - t0;
    const int sub = (n + NW - 1) / NW;
    const int w0 = min(t1, t0 + warp * sub), w1 = min(t1, w0 + sub);

    // ------------------------------------------------------------------ phase 1: layout
    int* wh = reinterpret_cast<int*>(smem + kBarBytes);   // [NW][ncols] per-warp histograms
    int* tot = wh + NW * ncols;                            // [ncols] CTA totals
    int* lb = tot + ncols;                                 // [ncols] sum over earlier CTAs
    for (int i = tid; i < (NW + 2) * ncols; i += blockDim.x) wh[i] = 0;
    for (int i = tid; i < n * F; i += blockDim.x) ws.tok_slot[(size_t)t0 * F + i] = -1;
    __syncthreads();

    {
        const int tpb = 32 / K;                 // tokens handled per warp step
        const int tl = lane / K, k = lane - tl * K;
        const bool lane_on = tl < tpb;
        const unsigned kmask = (K == 32) ? 0xffffffffu : ((1u << K) - 1u);
        const unsigned grp = lane_on ? (kmask << (tl * K)) : 0u;
        const unsigned lt = ptx::lanemask_lt();
        int* my = wh + warp * ncols;
        constexpr int U = 4;                    // steps whose ids are fetched together
        for (int tb0 = w0; tb0 < w1; tb0 += tpb * U) {
            long long idv[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int t = tb0 + u * tpb + tl;
                idv[u] = (lane_on && t < w1) ? a.ids[(size_t)t * K + k] : -1ll;
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int tb = tb0 + u * tpb;
                if (tb >= w1) break;            // warp-uniform
                const int t = tb + tl;
                const bool in = lane_on && t < w1;
                const long long id = idv[u];
                // Range check at full width, before narrowing to int.
                bool bad = in && (id < -1ll || id >= (long long)E);
                int e = (in && !bad && id >= 0) ? (int)id : -1;
                int key = (e >= 0) ? (tl * kMaxExperts + e) : -(lane + 1);
                unsigned peers = __match_any_sync(ptx::kFullMask, key);
                if (e >= 0 && __popc(peers) > 1) bad = true;      // expert repeated in a token
                const unsigned badmask = __ballot_sync(ptx::kFullMask, bad);
                if (bad) {
                    report(wc, kBadRoute, -1, ep, t, id, k, 0);
                    atomicAdd(&c.poison[kBadRoutes], 1);
                }
                if (badmask & grp) e = -1;      // an illegal token publishes nothing

                // rank of this choice among the warp's earlier choices of the same expert
                key = (e >= 0) ? e : -(lane + 1);
                peers = __match_any_sync(ptx::kFullMask, key);
                const int rank_e = __popc(peers & lt);
                int pos = -1;
                if (e >= 0) pos = my[F + e] + rank_e;
                __syncwarp();
                if (e >= 0 && rank_e == 0) my[F + e] += __popc(peers);

                // one record per (token, FFN rank): the lowest lane of the pair claims a slot
                const int f = (e >= 0) ? e / EL : -1;
                key = (e >= 0) ? (tl * 64 + f) : -(lane + 1);
                const unsigned ptf = __match_any_sync(ptx::kFullMask, key);
                const bool lead = (e >= 0) && ((ptf & lt) == 0u);
                key = lead ? f : -(lane + 1);
                const unsigned pf = __match_any_sync(ptx::kFullMask, key);
                const int rank_f = __popc(pf & lt);
                int slot = -1;
                if (lead) slot = my[f] + rank_f;
                __syncwarp();
                if (lead && rank_f == 0) my[f] += __popc(pf);
                __syncwarp();

                if (in) {
                    ws.route_e[(size_t)t * K + k] = e;
                    ws.route_pos[(size_t)t * K + k] = pos;
                }
                if (lead) ws.tok_slot[(size_t)t * F + f] = slot;
            }
        }
    }
    __syncthreads();

    // exclusive scan over the CTA's warps, publish the CTA aggregate
    for (int col = tid; col < ncols; col += blockDim.x) {
        int run = 0;
        for (int w = 0; w < NW; ++w) {
            const int v = wh[w * ncols + col];
            wh[w * ncols + col] = run;
            run += v;
        }
        tot[col] = run;
        ptx::st_relaxed_gpu_u64(&ws.agg[(size_t)cta * ncols + col],
                                ((unsigned long long)ep << 32) | (unsigned)run);
    }

    // decoupled look-back: sum the aggregates of all earlier CTAs
    {
        constexpr int U = 8;
        const int total = cta * ncols;
        bool ok = true;
        for (int base = tid; base < total && ok; base += blockDim.x * U) {
            unsigned long long v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int idx = base + u * blockDim.x;
                v[u] = (idx < total) ? ptx::ld_relaxed_gpu_u64(&ws.agg[idx]) : 0ull;
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int idx = base + u * blockDim.x;
                if (idx >= total) break;
                if ((unsigned)(v[u] >> 32) != ep) {
                    unsigned long long vv = v[u];
                    ok = spin_until(wc, [&] {
                        vv = ptx::ld_relaxed_gpu_u64(&ws.agg[idx]);
                        return (unsigned)(vv >> 32) == ep;
                    });
                    if (!ok) {
                        report(wc, kTimeoutLookback, idx / ncols, ep, ep, (long long)(vv >> 32), cta, 0);
                        poison(wc);
                        break;
                    }
                    v[u] = vv;
                }
                const int cnt = (int)(unsigned)v[u];
                if (cnt) atomicAdd(&lb[idx % ncols], cnt);
            }
        }
    }
    __syncthreads();

    // The last CTA now holds this source's totals: push them to the FFN ranks.
    if (cta == G - 1) {
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

    // fix-up: warp-local ranks -> global pos / slot
    {
        const int* my = wh + warp * ncols;
        const int cntk = (w1 - w0) * K;
        for (int i = lane; i < cntk; i += 32) {
            const size_t idx = (size_t)w0 * K + i;
            const int e = ws.route_e[idx];
            if (e >= 0) ws.route_pos[idx] += my[F + e] + lb[F + e];
        }
        const int cntf = (w1 - w0) * F;
        for (int i = lane; i < cntf; i += 32) {
            const size_t idx = (size_t)w0 * F + i;
            const int f = i % F;
            const int s = ws.tok_slot[idx];
            if (s >= 0) ws.tok_slot[idx] = s + my[f] + lb[f];
        }
    }
    // Shared memory changes hands from generic-proxy scratch to bulk-copy buffers.
    ptx::fence_proxy_async_smem();
    __syncthreads();

    // ------------------------------------------------------------------ phase 2: push
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    unsigned char* bufs = smem + kBarBytes + (size_t)warp * kNB * g.rec_bytes;
    if (lane == 0) {
        for (int b = 0; b < kNB; ++b) ptx::mbar_init(&bars[warp * kNB + b], 1);
        ptx::fence_mbar_init();
    }
    __syncwarp();

    const unsigned char* xb = static_cast<const unsigned char*>(a.x);
    const int sg = g.fp8 ? g.scale_groups : 0;
    int it = 0;
    int pend_slot = -1;
    unsigned pend_mask = 0;
    bool alive = true;
    for (int t = t0 + warp; t < t1 && alive; t += NW) {
        const int slot = (lane < F) ? ws.tok_slot[(size_t)t * F + lane] : -1;
        const unsigned mask = __ballot_sync(ptx::kFullMask, slot >= 0);
        if (mask == 0) continue;
        const int b = it % kNB;
        const unsigned parity = (it / kNB) & 1u;
        unsigned char* buf = bufs + (size_t)b * g.rec_bytes;
        uint64_t* bar = &bars[warp * kNB + b];
        if (lane == 0) {
            if (it >= kNB) ptx::bulk_wait_read<kNB - 1>();   // buffer's previous stores have read it
            ptx::mbar_expect_tx(bar, g.payload_bytes);
            ptx::bulk_load(buf, xb + (size_t)t * g.payload_bytes, g.payload_bytes, bar);
        }
        __syncwarp();
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
        __syncwarp();
        if (lane == 0) {
            // A local bulk load always completes; the bound only guards against a broken build.
            alive = spin_until(wc, [&] { return ptx::mbar_try_wait(bar, parity); });
        }
        alive = __shfl_sync(ptx::kFullMask, alive, 0);
        if (!alive) break;
        for (unsigned m = mask; m; m &= m - 1) {
            const int f = __ffs(m) - 1;
            const int s = __shfl_sync(ptx::kFullMask, slot, f);
            if (lane == 0) {
                const bool inb = !c.bounds_check || (s >= 0 && s < C);
                if (inb)
                    ptx::bulk_store(c.peer[f] + g.f_stage + ((size_t)ai * C + s) * g.rec_bytes, buf, g.rec_bytes);
                else
                    report(wc, kBadIndex, f, ep, C, s, t, 1);
            }
        }
        if (lane == 0) ptx::bulk_commit();
        // release the arrival flags of the previous token, whose stores have now completed
        if (pend_mask) {
            if (lane == 0) {
                ptx::bulk_wait<kNB - 1>();
                ptx::fence_acq_rel_sys();
            }
            for (unsigned m = pend_mask; m; m &= m - 1) {
                const int f = __ffs(m) - 1;
                const int s = __shfl_sync(ptx::kFullMask, pend_slot, f);
                if (lane == 0 && s >= 0 && s < C)
                    ptx::st_relaxed_sys(reinterpret_cast<uint32_t*>(c.peer[f] + g.f_slot_flag) + (size_t)ai * C + s, ep);
            }
        }
        pend_mask = mask;
        pend_slot = slot;
        ++it;
    }
    if (lane == 0) ptx::bulk_wait<0>();
    if (pend_mask && alive) {
        if (lane == 0) ptx::fence_acq_rel_sys();
        for (unsigned m = pend_mask; m; m &= m - 1) {
            const int f = __ffs(m) - 1;
            const int s = __shfl_sync(ptx::kFullMask, pend_slot, f);
            if (lane == 0 && s >= 0 && s < C)
                ptx::st_relaxed_sys(reinterpret_cast<uint32_t*>(c.peer[f] + g.f_slot_flag) + (size_t)ai * C + s, ep);
        }
    }

    // The last CTA to get here closes the exchange on this side.
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(&ws.ticket[0], 1u) == (unsigned)(G - 1)) {
            ws.ticket[0] = 0;
            ws.epoch[0] = ep;
            __threadfence();
        }
    }
}

}  // namespace

int max_dispatch_ctas() { return kMaxCtas; }

LaunchShape dispatch_shape(const Geometry& g, int tokens, int num_sms, int max_smem) {
    LaunchShape s{};
    const int ncols = g.ffn + g.num_experts;
    int warps = (max_smem - kBarBytes) / (kNB * g.rec_bytes);
    if (warps > kMaxWarps) warps = kMaxWarps;
    if (warps < 1) warps = 1;
    // Phase 1 scratch must fit too.
    while (warps > 1 && kBarBytes + (warps + 2) * ncols * 4 > max_smem) --warps;
    int ctas = num_sms < kMaxCtas ? num_sms : kMaxCtas;
    // No point in more CTAs than there are warp-sized groups of tokens.
    int want = (tokens + warps - 1) / warps;
    if (want < 1) want = 1;
    if (ctas > want) ctas = want;
    if (ctas < 1) ctas = 1;
    s.ctas = ctas;
    s.warps = warps;
    int p1 = kBarBytes + (warps + 2) * ncols * 4;
    int p2 = kBarBytes + warps * kNB * g.rec_bytes;
    s.smem_bytes = p1 > p2 ? p1 : p2;
    return s;
}

cudaError_t launch_dispatch(const RankCtx& c, const AttnWs& ws, const DispatchArgs& a, LaunchShape s,
                            cudaStream_t stream) {
    dispatch_kernel<<<s.ctas, s.warps * 32, s.smem_bytes, stream>>>(c, ws, a);
    return cudaGetLastError();
}

cudaError_t configure_dispatch(int max_smem) {
    return cudaFuncSetAttribute(dispatch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
}

}  // namespace afdep
