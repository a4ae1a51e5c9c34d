// Deterministic routing layout of one source rank, computed inside a running grid.
//
// Every CTA owns a contiguous chunk of tokens.  Its warps rank each (token, k) choice among
// the earlier choices of the same expert and each (token, FFN rank) record among the earlier
// records for that rank: first inside the warp's sub-range (match-any), then across the
// CTA's warps (shared-memory scan), then across CTAs (decoupled look-back over epoch-tagged
// aggregates in global scratch).  Outputs, final when the function returns:
//   route_e[t][k]   expert id or -1 (skipped, or the whole token was illegal)
//   route_pos[t][k] number of earlier choices of that expert by this source
//   tok_slot[t][f]  number of earlier tokens of this source with a record for FFN rank f, or -1
// and, in shared memory, the CTA's own totals `tot[col]` and the sum over earlier CTAs
// `lb[col]` (columns: [0, F) records per FFN rank, then one per expert), so the last CTA
// holds the source's totals.  Illegal routes (id outside [-1, E) at full 64-bit width, or an
// expert twice in one token) are reported, not trapped.
//
// Covers what the reference spreads over its notify warps, its deterministic prologue and
// its route guard (deep_ep/include/deep_ep/impls/dispatch.cuh:93-157,
// dispatch_deterministic_prologue.cuh, afdep_roles.cuh:11-33).
#pragma once
#include "layout.h"
#include "ptx.cuh"
#include "status.cuh"

namespace afdep {

struct RouteLayoutOut {
    int* route_e;
    int* route_pos;
    int* tok_slot;
};

// Shared-memory ints the function needs at `scratch`.
__host__ __device__ __forceinline__ int route_layout_scratch_ints(int warps, int ncols) { return (warps + 2) * ncols; }

// Returns false (uniformly for the CTA) if the look-back was abandoned.
__device__ __forceinline__ bool route_layout_phase(const long long* __restrict__ ids, int T, int K, int E, int EL, int F,
                                                    unsigned ep, unsigned long long* agg, const RouteLayoutOut& o,
                                                    int* scratch, const WaitCtx& wc, int** tot_out, int** lb_out) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, NW = blockDim.x >> 5;
    const int G = gridDim.x, cta = blockIdx.x;
    const int ncols = F + E;
    const int chunk = (T + G - 1) / G;
    const int t0 = min(T, cta * chunk), t1 = min(T, t0 + chunk);
    const int n = t1 - t0;
    const int sub = (n + NW - 1) / NW;
    const int w0 = min(t1, t0 + warp * sub), w1 = min(t1, w0 + sub);

    int* wh = scratch;              // [NW][ncols] per-warp histograms, later exclusive warp bases
    int* tot = wh + NW * ncols;     // [ncols] CTA totals
    int* lb = tot + ncols;          // [ncols] sum over earlier CTAs
    __shared__ int s_dead;
    *tot_out = tot;
    *lb_out = lb;
    for (int i = tid; i < (NW + 2) * ncols; i += blockDim.x) wh[i] = 0;
    for (int i = tid; i < n * F; i += blockDim.x) o.tok_slot[(size_t)t0 * F + i] = -1;
    if (tid == 0) s_dead = 0;
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
                idv[u] = (lane_on && t < w1) ? ids[(size_t)t * K + k] : -1ll;
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
                    atomicAdd(&wc.poison[kBadRoutes], 1);
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
                    o.route_e[(size_t)t * K + k] = e;
                    o.route_pos[(size_t)t * K + k] = pos;
                }
                if (lead) o.tok_slot[(size_t)t * F + f] = slot;
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
        ptx::st_relaxed_gpu_u64(&agg[(size_t)cta * ncols + col], ((unsigned long long)ep << 32) | (unsigned)run);
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
                v[u] = (idx < total) ? ptx::ld_relaxed_gpu_u64(&agg[idx]) : 0ull;
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int idx = base + u * blockDim.x;
                if (idx >= total) break;
                if ((unsigned)(v[u] >> 32) != ep) {
                    unsigned long long vv = v[u];
                    ok = spin_until(wc, [&] {
                        vv = ptx::ld_relaxed_gpu_u64(&agg[idx]);
                        return (unsigned)(vv >> 32) == ep;
                    });
                    if (!ok) {
                        report(wc, kTimeoutLookback, idx / ncols, ep, ep, (long long)(vv >> 32), cta, 0);
                        poison(wc);
                        s_dead = 1;
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

    // fix-up: warp-local ranks -> global pos / slot
    {
        const int* my = wh + warp * ncols;
        const int cntk = (w1 - w0) * K;
        for (int i = lane; i < cntk; i += 32) {
            const size_t idx = (size_t)w0 * K + i;
            const int e = o.route_e[idx];
            if (e >= 0) o.route_pos[idx] += my[F + e] + lb[F + e];
        }
        const int cntf = (w1 - w0) * F;
        for (int i = lane; i < cntf; i += 32) {
            const size_t idx = (size_t)w0 * F + i;
            const int f = i % F;
            const int s = o.tok_slot[idx];
            if (s >= 0) o.tok_slot[idx] = s + my[f] + lb[f];
        }
    }
    __syncthreads();
    return s_dead == 0;
}

}  // namespace afdep
