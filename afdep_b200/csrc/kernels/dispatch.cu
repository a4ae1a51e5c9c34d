// Attention-side dispatch: route guard, deterministic layout and payload push in ONE launch.
//
// Phase 1 (layout, route_layout.cuh) ranks every (token, k) choice among the earlier choices
// of the same expert and every (token, FFN rank) record among the earlier records for that
// rank, so placement depends only on the inputs.  Large batches split the tokens over the
// CTAs and join them with a decoupled look-back; decode-sized batches let every CTA rank all
// tokens itself, with no traffic between CTAs.  The CTA's part of the table stays in shared
// memory for phase 2.  The CTA that holds the source's totals pushes them to the FFN ranks
// (the count "all-to-all") from its flag warp, ahead of the payload flags.
//
// Phase 2 (push) — one data warp per token over a ring of record buffers: a bulk async copy
// brings the row into shared memory once, lanes append scales/routes/weights, and one bulk
// store per destination FFN rank writes the finished record straight into that rank's staging
// slot over NVLink.  Once a store group has completed, the data warp hands the token to the
// CTA's flag warp, which issues the system-scope fence and the 4-byte arrival flag per record;
// the receiver can start on a record as soon as it has landed, and the (slow) fence never
// stalls a data warp.
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

constexpr int kBarBytes = 1024;   // mbarriers and hand-off counters at the start of dynamic shared memory
constexpr int kMaxWarps = 16;
constexpr unsigned kFlagPatience = 8;   // polls a flag warp holds back a fence for stragglers
constexpr int kMaxCtas = 160;
constexpr int kMaxRouteBytes = 64 * 1024;   // largest routing table kept in shared memory
constexpr int kRedundantEntries = 4096;     // every CTA ranks all tokens up to this many (token, k) pairs

// How a launch is laid out; computed on the host, identical for every CTA.
struct DispatchPlan {
    int ctas, warps, nb, smem_bytes;
    int data_warps;      // warps [0, data_warps) push records, warp data_warps releases flags, the
                         // rest only help with the layout phase
    int route_rows;      // rows of the shared-memory routing table, 0: keep it in global memory
    int redundant;       // 1: every CTA ranks all tokens (no traffic between CTAs)
    int route_bytes;     // bytes reserved for the table
    int totals_bytes;    // bytes reserved for tot/lb
};

// NB record buffers per data warp form a ring: while token i is being stored, token i+1 is
// already loading, and token i-(NB-2) is handed to the flag warp once its store group has
// completed.  NB = 2 degenerates to load -> store -> wait -> hand off.
template <int NB>
__global__ void __launch_bounds__(kMaxWarps * 32, 1)
dispatch_kernel(const RankCtx c, const AttnWs ws, const DispatchArgs a, const DispatchPlan plan) {
    constexpr int L = NB - 2;     // how many tokens the hand-off lags behind the stores
    extern __shared__ __align__(128) unsigned char smem[];
    const Geometry& g = c.g;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = gridDim.x, cta = blockIdx.x;
    const int F = g.ffn, K = g.top_k, E = g.num_experts, EL = g.experts_local, C = g.capacity;
    const int ncols = F + E, LW = 2 * K + F;
    const int ai = c.role_rank;
    const unsigned ep = ptx::ld_acquire_gpu(&ws.epoch[0]) + 1u;
    const WaitCtx wc{c.status, c.poison, c.budget, c.rank, /*kernel=*/1};
    trace_stamp(c.trace, kTraceDispatch, 0);

    const int T = a.T;

    // shared memory: [bars | routing table | totals | overlay: layout histograms, then record buffers]
    int* local = plan.route_rows ? reinterpret_cast<int*>(smem + kBarBytes) : nullptr;
    int* tot = reinterpret_cast<int*>(smem + kBarBytes + plan.route_bytes);
    int* lb = tot + ncols;
    unsigned char* overlay = smem + kBarBytes + plan.route_bytes + plan.totals_bytes;

    // ------------------------------------------------------------------ phase 1: layout
    RouteLayoutJob job;
    job.ids = a.ids;
    job.ids32 = a.ids32;
    job.T = T;
    job.K = K;
    job.E = E;
    job.EL = EL;
    job.F = F;
    job.ep = ep;
    job.agg = ws.agg;
    job.out = RouteLayoutOut{plan.redundant ? nullptr : ws.route_e, plan.redundant ? nullptr : ws.route_pos, ws.tok_slot};
    job.wh = reinterpret_cast<int*>(overlay);
    job.tot = tot;
    job.lb = lb;
    job.local = local;
    job.redundant = plan.redundant;
    job.trace = c.trace;
    const bool alive = route_layout_phase(job, wc);
    // Phase 2 walks the tokens round-robin over all CTAs (so records reach the receivers in
    // slot order).  When the layout is distributed, a token's routing words were produced by
    // the CTA that owns its chunk: publish "my chunk is final" for the others to wait on.
    if (!plan.redundant) {
        __threadfence();
        __syncthreads();
        if (tid == 0) ptx::st_release_gpu(&ws.chunk_done[cta], alive ? ep : 0u);
    }
    // Shared memory changes hands from generic-proxy scratch to bulk-copy buffers.
    ptx::fence_proxy_async_smem();

    // ------------------------------------------------------------------ phase 2: push
    // Warps [0, ND) move data, warp ND releases counts and arrival flags; any further warps only
    // took part in the layout phase (more hands there shorten the part every exchange waits on).
    const int ND = plan.data_warps;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    int* done_cnt = reinterpret_cast<int*>(smem + kBarBytes - 128);   // [ND] tokens completed per data warp
    unsigned char* bufs = overlay + (size_t)warp * NB * g.rec_bytes;
    if (warp < ND && lane == 0) {
        for (int b = 0; b < NB; ++b) ptx::mbar_init(&bars[warp * NB + b], 1);
        ptx::fence_mbar_init();
    }
    if (tid < 32) done_cnt[tid] = 0;
    __syncthreads();
    trace_stamp(c.trace, kTraceDispatch, 1);

    const unsigned char* xb = static_cast<const unsigned char*>(a.x);
    const int sg = g.fp8 ? g.scale_groups : 0;
    // Token j of data warp w in this CTA: consecutive tokens go to consecutive warps of
    // consecutive CTAs, so the whole grid sweeps the batch front to back.
    const int tok_stride = G * ND;
    auto token_of = [&](int w, int j) { return (j * G + cta) * ND + w; };
    auto tokens_of = [&](int w) { return (alive && token_of(w, 0) < T) ? (T - token_of(w, 0) + tok_stride - 1) / tok_stride : 0; };
    const bool use_local = plan.redundant != 0;      // the shared-memory table covers every token
    const int chunk = (T + G - 1) / G;
    auto local_row = [&](int t) { return local + (size_t)t * LW; };
    auto slot_of = [&](int t, int f) { return use_local ? local_row(t)[2 * K + f] : ws.tok_slot[(size_t)t * F + f]; };

    if (warp < ND) {
        const int n_w = tokens_of(warp);
        unsigned phase_bits = 0;      // lane 0: parity of each buffer's mbarrier
        int ready_upto = use_local ? G : 0;          // chunks [0, ready_upto) are known to be final
        bool ok = true;

        // A(i): start loading token i into its ring buffer and append its metadata.
        auto stage = [&](int i, int& slot, unsigned& mask) {
            const int t = token_of(warp, i);
            const int owner = t / chunk;
            if (owner >= ready_upto) {               // warp-uniform: wait for the owner's layout
                bool fin = true;
                if (lane == 0) {
                    unsigned seen = 0;
                    fin = spin_until(wc, [&] {
                        seen = ptx::ld_acquire_gpu(&ws.chunk_done[owner]);
                        return seen == ep;
                    });
                    if (!fin) {
                        report(wc, kTimeoutLookback, owner, ep, ep, seen, cta, 2);
                        poison(wc);
                    }
                }
                fin = __shfl_sync(ptx::kFullMask, fin, 0);
                if (!fin) {
                    ok = false;
                    slot = -1;
                    mask = 0;
                    return;
                }
                ready_upto = owner + 1;
            }
            slot = (lane < F) ? slot_of(t, lane) : -1;
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
                if (use_local) {
                    const int* row = local_row(t);
                    meta[lane] = row[lane];
                    meta[K + lane] = row[K + lane];
                } else {
                    meta[lane] = ws.route_e[(size_t)t * K + lane];
                    meta[K + lane] = ws.route_pos[(size_t)t * K + lane];
                }
                reinterpret_cast<float*>(meta)[2 * K + lane] = a.weights[(size_t)t * K + lane];
            }
            if (lane == 0) meta[3 * K] = t;
            for (int gi = lane; gi < sg; gi += 32)
                reinterpret_cast<float*>(buf + g.payload_bytes)[gi] = a.x_scale[(size_t)t * a.ss0 + (size_t)gi * a.ss1];
            ptx::fence_proxy_async_smem();
        };

        int slot_c = -1, slot_n = -1;
        unsigned mask_c = 0, mask_n = 0;
        if (n_w > 0) stage(0, slot_c, mask_c);
        for (int i = 0; i < n_w && ok; ++i) {
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
                const int t = token_of(warp, i);
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
                    if (a.flag_mode == 1) {
                        ptx::fence_proxy_async_global();
                        const int tj = token_of(warp, i - L);
                        for (int f = 0; f < F; ++f) {
                            const int sj = slot_of(tj, f);
                            if (sj >= 0 && sj < C)
                                ptx::st_relaxed_sys(reinterpret_cast<uint32_t*>(c.peer[f] + g.f_slot_flag) + (size_t)ai * C + sj, ep);
                        }
                    }
                    ptx::st_release_cta_shared(&done_cnt[warp], i - L + 1);
                }
            }
            slot_c = slot_n;
            mask_c = mask_n;
        }
        if (lane == 0) {
            ptx::bulk_wait<0>();
            if (a.flag_mode == 1 && ok) {
                ptx::fence_proxy_async_global();
                for (int j = (n_w > L ? n_w - L : 0); j < n_w; ++j) {
                    const int tj = token_of(warp, j);
                    for (int f = 0; f < F; ++f) {
                        const int sj = slot_of(tj, f);
                        if (sj >= 0 && sj < C)
                            ptx::st_relaxed_sys(reinterpret_cast<uint32_t*>(c.peer[f] + g.f_slot_flag) + (size_t)ai * C + sj, ep);
                    }
                }
            }
            ptx::st_release_cta_shared(&done_cnt[warp], ok ? n_w : -1);
        }
    } else if (warp == ND) {
        // Flag warp.  First, in the CTA that holds the source's totals, the count "all-to-all":
        // per-expert counts and the record count go to every FFN rank, each packed with the
        // epoch into one 8-byte word.  The word is its own arrival flag, so no fence is needed
        // and the receivers can lay out their rows as soon as the words land.
        if (cta == G - 1 && alive) {
            const int cs = cnt_stride(g);
            for (int idx = lane; idx < F * (EL + 1); idx += 32) {
                const int f = idx / (EL + 1), el = idx - f * (EL + 1);
                const int col = (el < EL) ? (F + f * EL + el) : f;
                unsigned long long* dst = reinterpret_cast<unsigned long long*>(c.peer[f] + g.f_cnt) + (size_t)ai * cs + el;
                ptx::st_relaxed_sys_u64(dst, ((unsigned long long)ep << 32) | (unsigned)(lb[col] + tot[col]));
            }
            __syncwarp();
            if (lane == 0) trace_stamp_here(c.trace, kTraceDispatch, 3);    // counts released
        }
        // Then lane w follows data warp w: one system-scope fence covers every token handed
        // over since the last one, so the fence never stalls a data warp.  A fence costs
        // microseconds while remote stores are in flight, so the warp waits (briefly) until every
        // data warp that still owes flags has something new before it pays for one.
        const int mine = (lane < ND) ? tokens_of(lane) : 0;
        int flagged = 0;
        bool aborted = false;
        const long long t_begin = clock64();
        unsigned idle = 0, patience = 0;
        while (true) {
            int d = (lane < ND && !aborted) ? ptx::ld_acquire_cta_shared(&done_cnt[lane]) : flagged;
            if (d < 0) {
                aborted = true;
                d = flagged;
            }
            if (d > flagged && a.flag_mode == 1) flagged = d;      // the data warps already did it
            const unsigned fresh = __ballot_sync(ptx::kFullMask, d > flagged);
            const unsigned owing = __ballot_sync(ptx::kFullMask, lane < ND && !aborted && flagged < mine);
            if (fresh != 0 && (fresh == owing || ++patience > kFlagPatience)) {
                patience = 0;
                if (d > flagged) {
                    ptx::fence_acq_rel_sys();
                    for (int j = flagged; j < d; ++j) {
                        const int t = token_of(lane, j);
                        for (int f = 0; f < F; ++f) {
                            const int s = slot_of(t, f);
                            if (s >= 0 && s < C)
                                ptx::st_relaxed_sys(reinterpret_cast<uint32_t*>(c.peer[f] + g.f_slot_flag) + (size_t)ai * C + s, ep);
                        }
                    }
                    flagged = d;
                }
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

int align128(int v) { return (v + 127) / 128 * 128; }

DispatchPlan plan_dispatch(const Geometry& g, int tokens, int num_sms) {
    DispatchPlan p{};
    const int ncols = g.ffn + g.num_experts;
    const int LW = 2 * g.top_k + g.ffn;
    const int avail = g_dyn_smem - kBarBytes;
    p.totals_bytes = align128(2 * ncols * 4);
    // Ring depth from the record size alone: the deepest that keeps enough warps per CTA.
    const int room = avail - p.totals_bytes;
    p.nb = (room / (4 * g.rec_bytes) >= 6) ? 4 : (room / (3 * g.rec_bytes) >= 3) ? 3 : 2;
    int data_warps = room / (p.nb * g.rec_bytes);
    if (data_warps > kMaxWarps - 1) data_warps = kMaxWarps - 1;
    if (data_warps < 1) data_warps = 1;
    int ctas = num_sms < kMaxCtas ? num_sms : kMaxCtas;
    int want = (tokens + data_warps - 1) / data_warps;   // no more CTAs than warp-sized groups of tokens
    if (want < 1) want = 1;
    if (ctas > want) ctas = want;
    if (ctas < 1) ctas = 1;
    p.ctas = ctas;
    // Routing table in shared memory when it is small enough.
    const int chunk = (tokens + ctas - 1) / ctas;
    p.redundant = (tokens * g.top_k <= kRedundantEntries && tokens * LW * 4 <= kMaxRouteBytes && ctas > 1) ? 1 : 0;
    const int rows = p.redundant ? tokens : chunk;
    if (rows > 0 && rows * LW * 4 <= kMaxRouteBytes) {
        p.route_rows = rows;
        p.route_bytes = align128(rows * LW * 4);
    } else {
        p.redundant = 0;
    }
    data_warps = (room - p.route_bytes) / (p.nb * g.rec_bytes);
    if (data_warps > kMaxWarps - 1) data_warps = kMaxWarps - 1;
    if (data_warps < 1) data_warps = 1;
    p.data_warps = data_warps;
    // Always a full block: the warps beyond the data warps and the flag warp join the layout
    // phase.  The layout histograms share the overlay with the record buffers.
    int warps = kMaxWarps;
    while (warps > data_warps + 1 && p.route_bytes + p.totals_bytes + warps * ncols * 4 > avail) --warps;
    while (warps > 2 && p.route_bytes + p.totals_bytes + warps * ncols * 4 > avail) {
        --warps;
        p.data_warps = warps - 1;
    }
    p.warps = warps;
    const int p1 = warps * ncols * 4;
    const int p2 = p.data_warps * p.nb * g.rec_bytes;
    p.smem_bytes = kBarBytes + p.route_bytes + p.totals_bytes + (p1 > p2 ? p1 : p2);
    return p;
}

}  // namespace

int max_dispatch_ctas() { return kMaxCtas; }

LaunchShape dispatch_shape(const Geometry& g, int tokens, int num_sms, int max_smem) {
    (void)max_smem;
    const DispatchPlan p = plan_dispatch(g, tokens, num_sms);
    return LaunchShape{p.ctas, p.warps, p.smem_bytes};
}

cudaError_t launch_dispatch(const RankCtx& c, const AttnWs& ws, const DispatchArgs& a, LaunchShape s,
                            cudaStream_t stream) {
    const DispatchPlan p = plan_dispatch(c.g, a.T, s.ctas);
    const void* fn = p.nb == 4 ? reinterpret_cast<const void*>(dispatch_kernel<4>)
                   : p.nb == 3 ? reinterpret_cast<const void*>(dispatch_kernel<3>)
                               : reinterpret_cast<const void*>(dispatch_kernel<2>);
    void* params[] = {const_cast<RankCtx*>(&c), const_cast<AttnWs*>(&ws), const_cast<DispatchArgs*>(&a), const_cast<DispatchPlan*>(&p)};
    // With the layout split over the CTAs, a CTA waits on the look-back aggregates and on the
    // "chunk final" words of other CTAs, so all of them must be on the GPU together.  A
    // cooperative launch guarantees that (it starts only when the whole grid fits beside what is
    // already running, and a grid that can never fit is refused here, on the host) -- the
    // reference launches its dispatch the same way (csrc/kernels/elastic/dispatch.hpp:306).
    // When every CTA ranks all tokens itself there is nothing to wait for and a plain launch does.
    if (!p.redundant && p.ctas > 1)
        return cudaLaunchCooperativeKernel(fn, dim3(p.ctas), dim3(p.warps * 32), params, (size_t)p.smem_bytes, stream);
    return cudaLaunchKernel(fn, dim3(p.ctas), dim3(p.warps * 32), params, (size_t)p.smem_bytes, stream);
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
