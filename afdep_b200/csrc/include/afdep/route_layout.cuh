// Deterministic routing layout of one source rank, computed inside a running grid.
//
// Every (token, k) choice is ranked among the earlier choices of the same expert and every
// (token, FFN rank) record among the earlier records for that rank, in token order:
//   route_e[t][k]   expert id or -1 (skipped, or the whole token was illegal)
//   route_pos[t][k] number of earlier choices of that expert by this source
//   tok_slot[t][f]  number of earlier tokens of this source with a record for FFN rank f, or -1
// plus the source's totals per column (columns: [0, F) records per FFN rank, then one per
// expert).  Illegal routes (id outside [-1, E) at full 64-bit width, or an expert twice in
// one token) are reported, not trapped, and publish nothing.
//
// Two ways to split the work:
//   distributed  every CTA owns a contiguous chunk of tokens; warps rank inside their
//                sub-range (shuffle compares inside a token, one token at a time on the
//                warp's counters), a shared-memory scan joins the warps, a decoupled
//                look-back over epoch-tagged aggregates in global scratch joins the CTAs.
//   redundant    for small inputs every CTA ranks ALL tokens itself and keeps the part it
//                owns: no traffic between CTAs at all, which is what decode-sized batches want.
// Results for the CTA's own tokens can stay in a shared-memory table (`local`), so the caller's
// next phase reads them without a trip through global memory; global outputs are written once.
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
    int* route_e;     // may be null when the caller keeps the table in shared memory
    int* route_pos;   // may be null, as above
    int* tok_slot;
};

struct RouteLayoutJob {
    const long long* ids;        // int64 ids [T][K], or null when ids32 is used
    const int* ids32 = nullptr;  // int32 ids [T][K] (the reference's 32-bit index build, compiled.cuh:54-72)
    int T, K, E, EL, F;
    unsigned ep;                 // tag of this launch in the aggregate array
    unsigned long long* agg;     // [gridDim.x][F + E], distributed mode only
    RouteLayoutOut out;
    int* wh;                     // smem [warps][F + E]
    int* tot;                    // smem [F + E]: this CTA's totals
    int* lb;                     // smem [F + E]: sum over earlier CTAs (zero in redundant mode)
    int* local;                  // smem [tokens][2K + F] (e, pos, slot) or null
    int redundant;               // 1: every CTA ranks all tokens
    unsigned long long* trace;   // optional time stamps (row 4 of the trace buffer), or null
};

__host__ __device__ __forceinline__ int route_layout_scratch_ints(int warps, int ncols) { return (warps + 2) * ncols; }

// Token range a CTA owns.
__device__ __forceinline__ void route_layout_chunk(int T, int& t0, int& t1) {
    const int G = gridDim.x;
    const int chunk = (T + G - 1) / G;
    t0 = min(T, (int)blockIdx.x * chunk);
    t1 = min(T, t0 + chunk);
}

// Row of the shared-memory table that holds token t.
__device__ __forceinline__ int route_layout_local_row(const RouteLayoutJob& j, int t, int t0) {
    return j.redundant ? t : t - t0;
}

// Returns false (uniformly for the CTA) if the look-back was abandoned.  On return the CTA
// holds totals in tot/lb (the last CTA of a distributed run, every CTA of a redundant run,
// has the source's totals as lb + tot).
__device__ __forceinline__ bool route_layout_phase(const RouteLayoutJob& j, const WaitCtx& wc) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, NW = blockDim.x >> 5;
    const int cta = blockIdx.x;
    const int T = j.T, K = j.K, E = j.E, EL = j.EL, F = j.F;
    const int ncols = F + E;
    const int LW = 2 * K + F;                 // ints per row of the local table
    int t0, t1;
    route_layout_chunk(T, t0, t1);
    // range this CTA ranks, and the part of it this warp ranks
    const int r0 = j.redundant ? 0 : t0, r1 = j.redundant ? T : t1;
    const int n = r1 - r0;
    const int sub = (n + NW - 1) / NW;
    const int w0 = min(r1, r0 + warp * sub), w1 = min(r1, w0 + sub);

    int* wh = j.wh;
    __shared__ int s_dead;
    for (int i = tid; i < NW * ncols; i += blockDim.x) wh[i] = 0;
    for (int i = tid; i < ncols; i += blockDim.x) {
        j.tot[i] = 0;
        j.lb[i] = 0;
    }
    if (j.local != nullptr) {
        for (int i = tid; i < n * F; i += blockDim.x) j.local[(i / F) * LW + 2 * K + (i % F)] = -1;
    } else {
        for (int i = tid; i < n * F; i += blockDim.x) j.out.tok_slot[(size_t)r0 * F + i] = -1;
    }
    if (tid == 0) s_dead = 0;
    __syncthreads();
    trace_stamp(j.trace, 4, 0);

    {
        const int tpb = 32 / K;                 // tokens handled per warp step
        const int tl = lane / K, k = lane - tl * K;
        const bool lane_on = tl < tpb;
        const unsigned kmask = (K == 32) ? 0xffffffffu : ((1u << K) - 1u);
        const unsigned grp = lane_on ? (kmask << (tl * K)) : 0u;
        int* my = wh + warp * ncols;
        constexpr int U = 4;                    // steps whose ids are fetched together
        for (int tb0 = w0; tb0 < w1; tb0 += tpb * U) {
            long long idv[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int t = tb0 + u * tpb + tl;
                idv[u] = !(lane_on && t < w1) ? -1ll : (j.ids32 != nullptr ? (long long)j.ids32[(size_t)t * K + k] : j.ids[(size_t)t * K + k]);
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
                int f = (e >= 0) ? e / EL : -1;
                // Compare against the token's other choices (K - 1 shuffles): an expert chosen
                // twice makes the token illegal; the lowest k of an FFN rank leads its record.
                // (match.any would do this in one instruction, but its cost grows with the number
                // of distinct keys, and here nearly all 32 are distinct.)
                bool lead = e >= 0;
                for (int d = 1; d < K; ++d) {
                    int sk = k + d;
                    if (sk >= K) sk -= K;
                    const int src = (tl * K + sk) & 31;
                    const int oe = __shfl_sync(ptx::kFullMask, e, src);
                    const int of = __shfl_sync(ptx::kFullMask, f, src);
                    if (e >= 0 && oe == e) bad = true;
                    if (sk < k && of == f) lead = false;
                }
                const unsigned badmask = __ballot_sync(ptx::kFullMask, bad);
                if (bad && (!j.redundant || cta == 0)) {
                    report(wc, kBadRoute, -1, j.ep, t, id, k, 0);
                    atomicAdd(&wc.poison[kBadRoutes], 1);
                }
                if (badmask & grp) {            // an illegal token publishes nothing
                    e = -1;
                    f = -1;
                }
                lead = lead && e >= 0;
                // Ranks: one token at a time, so no two lanes ever touch the same counter (a legal
                // token names every expert, hence every FFN-rank leader, at most once).
                int pos = -1, slot = -1;
                for (int s = 0; s < tpb; ++s) {
                    if (tl == s && e >= 0) {
                        pos = my[F + e];
                        my[F + e] = pos + 1;
                    }
                    if (tl == s && lead) {
                        slot = my[f];
                        my[f] = slot + 1;
                    }
                    __syncwarp();
                }

                if (j.local != nullptr) {
                    int* row = j.local + (size_t)(t - r0) * LW;
                    if (in) {
                        row[k] = e;
                        row[K + k] = pos;
                    }
                    if (lead) row[2 * K + f] = slot;
                } else {
                    if (in) {
                        j.out.route_e[(size_t)t * K + k] = e;
                        j.out.route_pos[(size_t)t * K + k] = pos;
                    }
                    if (lead) j.out.tok_slot[(size_t)t * F + f] = slot;
                }
            }
        }
    }
    __syncthreads();
    trace_stamp(j.trace, 4, 1);

    // exclusive scan over the CTA's warps; in distributed mode publish the CTA aggregate
    for (int col = tid; col < ncols; col += blockDim.x) {
        int run = 0;
        for (int w = 0; w < NW; ++w) {
            const int v = wh[w * ncols + col];
            wh[w * ncols + col] = run;
            run += v;
        }
        j.tot[col] = run;
        if (!j.redundant)
            ptx::st_relaxed_gpu_u64(&j.agg[(size_t)cta * ncols + col], ((unsigned long long)j.ep << 32) | (unsigned)run);
    }

    // decoupled look-back: sum the aggregates of all earlier CTAs
    if (!j.redundant) {
        constexpr int U = 8;
        const int total = cta * ncols;
        bool ok = true;
        for (int base = tid; base < total && ok; base += blockDim.x * U) {
            unsigned long long v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int idx = base + u * blockDim.x;
                v[u] = (idx < total) ? ptx::ld_relaxed_gpu_u64(&j.agg[idx]) : 0ull;
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int idx = base + u * blockDim.x;
                if (idx >= total) break;
                if ((unsigned)(v[u] >> 32) != j.ep) {
                    unsigned long long vv = v[u];
                    ok = spin_until(wc, [&] {
                        vv = ptx::ld_relaxed_gpu_u64(&j.agg[idx]);
                        return (unsigned)(vv >> 32) == j.ep;
                    });
                    if (!ok) {
                        report(wc, kTimeoutLookback, idx / ncols, j.ep, j.ep, (long long)(vv >> 32), cta, 0);
                        poison(wc);
                        s_dead = 1;
                        break;
                    }
                    v[u] = vv;
                }
                const int cnt = (int)(unsigned)v[u];
                if (cnt) atomicAdd(&j.lb[idx % ncols], cnt);
            }
        }
    }
    __syncthreads();
    trace_stamp(j.trace, 4, 2);

    // fix-up: warp-local ranks -> global pos / slot, for the tokens this warp ranked
    {
        const int* my = wh + warp * ncols;
        const int* lb = j.lb;
        if (j.local != nullptr) {
            // lanes cover the pos and slot words of several tokens per step; the lane -> (token,
            // word) split is computed once, so the loop itself has no divisions
            const int per = LW - K;                          // words to fix per token
            const int tps = per <= 32 ? 32 / per : 1;        // tokens per step
            const int tsub = per <= 32 ? lane / per : 0;
            const int c0 = K + (per <= 32 ? lane - tsub * per : lane);
            if (tsub < tps) {
                for (int t = w0 + tsub; t < w1; t += tps) {
                    int* row = j.local + (size_t)(t - r0) * LW;
                    for (int c = c0; c < LW; c += (per <= 32 ? LW : 32)) {
                        if (c < 2 * K) {
                            const int e = row[c - K];
                            if (e >= 0) row[c] += my[F + e] + lb[F + e];
                        } else {
                            const int f = c - 2 * K;
                            if (row[c] >= 0) row[c] += my[f] + lb[f];
                        }
                    }
                }
            }
        } else {
            const int cntk = (w1 - w0) * K;
            for (int i = lane; i < cntk; i += 32) {
                const size_t idx = (size_t)w0 * K + i;
                const int e = j.out.route_e[idx];
                if (e >= 0) j.out.route_pos[idx] += my[F + e] + lb[F + e];
            }
            const int cntf = (w1 - w0) * F;
            for (int i = lane; i < cntf; i += 32) {
                const size_t idx = (size_t)w0 * F + i;
                const int f = i % F;
                const int s = j.out.tok_slot[idx];
                if (s >= 0) j.out.tok_slot[idx] = s + my[f] + lb[f];
            }
        }
    }
    __syncthreads();
    trace_stamp(j.trace, 4, 3);

    // the shared-memory table is final: write the global copies of the tokens this CTA owns
    if (j.local != nullptr) {
        const int own = t1 - t0;
        for (int i = tid; i < own * F; i += blockDim.x) {
            const int t = t0 + i / F, f = i % F;
            j.out.tok_slot[(size_t)t * F + f] = j.local[(size_t)route_layout_local_row(j, t, t0) * LW + 2 * K + f];
        }
        if (j.out.route_e != nullptr) {
            for (int i = tid; i < own * K; i += blockDim.x) {
                const int t = t0 + i / K, k = i % K;
                const int* row = j.local + (size_t)route_layout_local_row(j, t, t0) * LW;
                j.out.route_e[(size_t)t * K + k] = row[k];
                j.out.route_pos[(size_t)t * K + k] = row[K + k];
            }
        }
    }
    return s_dead == 0;
}

}  // namespace afdep
