// FFN-side kernels: receive (wait, place, expand) and reply (pre-reduce, publish).
//
// receive — every CTA first derives the exchange's row layout from the count vectors the
// sources pushed (bounded wait on one epoch flag per source): per-expert totals, aligned
// segment starts, `ends[]`, and the first row of every (source, expert) pair.  Then warps
// take wire records (source, slot) one at a time: poll the record's 4-byte arrival flag,
// pull the record into shared memory with one bulk copy, and write the payload once per
// local expert the token chose, at row_base[source][expert] + pos — a placement the sender
// already made deterministic, so no atomics and no second pass.  Expansion traffic stays in
// local HBM; NVLink carried the row only once per (token, FFN rank).
//
// reply — one warp per record again: sum the token's local expert rows (fp32 accumulate in
// top-k order, one rounding to BF16; a single row is copied bit-exactly) into the reply slot
// the attention rank will pull from, then release that rank's flag for the slot.
//
// Together they replace the reference's dispatch_copy_epilogue_impl, the sender half of
// combine_impl and the host's CPU polling loop (deep_ep/include/deep_ep/impls/
// dispatch_copy_epilogue.cuh, combine.cuh; csrc/elastic/buffer.hpp:994-1041).
#include <cuda_bf16.h>

#include "afdep/ffn_layout.cuh"
#include "afdep/kernels.h"
#include "afdep/status.cuh"

namespace afdep {

namespace {

constexpr int kBarBytes = 512;
constexpr int kMaxWarps = 16;

__device__ __forceinline__ int align_up_dev(int v, int a) { return (v + a - 1) / a * a; }

// Runs in every CTA of the receive kernel (and alone in the layout kernel).  Returns false,
// uniformly for the CTA, if a source's counts never arrived.
//
// A source publishes each count as one 8-byte word (epoch << 32 | count), which is its own
// arrival flag: a thread fetches a batch of words with independent loads and spins (bounded)
// only on those that do not carry this exchange's epoch yet.  The raw counts are parked in
// row_base / rec_prefix and turned into prefix sums in place.
__device__ bool compute_layout(const RankCtx& c, const WaitCtx& wc, unsigned ep, LayoutSmem& L) {
    const Geometry& g = c.g;
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int A = g.attn, EL = g.experts_local, cs = cnt_stride(g);
    unsigned char* heap = reinterpret_cast<unsigned char*>(c.peer[c.rank]);
    const unsigned long long* cnt = reinterpret_cast<const unsigned long long*>(heap + g.f_cnt);
    if (tid == 0) L.dead = 0;
    __syncthreads();
    constexpr int kBatch = 8;
    const int nwords = A * (EL + 1);
    for (int base = tid; base < nwords; base += kBatch * nthr) {
        unsigned long long v[kBatch];
#pragma unroll
        for (int q = 0; q < kBatch; ++q) {
            const int idx = base + q * nthr;
            if (idx < nwords) {
                const int a = idx / (EL + 1), el = idx - a * (EL + 1);
                v[q] = ptx::ld_relaxed_sys_u64(cnt + (size_t)a * cs + el);
            }
        }
#pragma unroll
        for (int q = 0; q < kBatch; ++q) {
            const int idx = base + q * nthr;
            if (idx >= nwords) continue;
            const int a = idx / (EL + 1), el = idx - a * (EL + 1);
            unsigned long long w = v[q];
            if ((unsigned)(w >> 32) != ep) {
                const unsigned long long* src = cnt + (size_t)a * cs + el;
                const bool ok = spin_until(wc, [&] {
                    w = ptx::ld_relaxed_sys_u64(src);
                    return (unsigned)(w >> 32) == ep;
                });
                if (!ok) {
                    report(wc, kTimeoutCounts, g.ffn + a, ep, ep, (long long)(w >> 32), el);
                    poison(wc);
                    L.dead = 1;
                    w = 0;
                }
            }
            const int n = (int)(unsigned)(w & 0xffffffffull);
            if (el < EL)
                L.row_base[a * EL + el] = n;
            else
                L.rec_prefix[a + 1] = n;
        }
    }
    __syncthreads();
    if (L.dead) return false;
    trace_stamp(c.trace, kTraceReceive, 3);     // counts of every source have arrived

    for (int el = tid; el < EL; el += nthr) {
        int t = 0;
        for (int a = 0; a < A; ++a) t += L.row_base[a * EL + el];
        L.tot[el] = t;
    }
    __syncthreads();
    if (tid < 32) {
        // exclusive scan of the aligned totals, a contiguous run of experts per lane
        const int per = (EL + 31) / 32;
        const int lo = min(EL, tid * per), hi = min(EL, lo + per);
        int sum = 0;
        for (int el = lo; el < hi; ++el) sum += align_up_dev(L.tot[el], g.alignment);
        int inc = sum;
        for (int d = 1; d < 32; d <<= 1) {
            const int v = __shfl_up_sync(ptx::kFullMask, inc, d);
            if (tid >= d) inc += v;
        }
        int run = inc - sum;
        for (int el = lo; el < hi; ++el) {
            L.start[el] = run;
            run += align_up_dev(L.tot[el], g.alignment);
        }
    }
    if (tid == 32 || (nthr <= 32 && tid == 0)) {
        int run = 0;      // rec_prefix[a + 1] holds source a's record count; make it a prefix sum in place
        for (int a = 0; a < A; ++a) {
            const int n = L.rec_prefix[a + 1];
            L.rec_prefix[a] = run;
            run += n;
        }
        L.rec_prefix[A] = run;
    }
    __syncthreads();
    for (int el = tid; el < EL; el += nthr) {
        int run = L.start[el];
        for (int a = 0; a < A; ++a) {
            const int n = L.row_base[a * EL + el];
            L.row_base[a * EL + el] = run;
            run += n;
        }
    }
    __syncthreads();
    return true;
}

__device__ void publish_layout(const RankCtx& c, const FfnWs& ws, const ReceiveArgs& r, const LayoutSmem& L) {
    const Geometry& g = c.g;
    const int A = g.attn, EL = g.experts_local;
    for (int el = threadIdx.x; el < EL; el += blockDim.x) {
        const int end = L.start[el] + L.tot[el];
        if (r.psum) r.psum[el] = end;
        if (r.expert_stats) r.expert_stats[el] += L.tot[el];     // one CTA publishes per exchange
        ws.ends[el] = end;
    }
    for (int i = threadIdx.x; i < A * EL; i += blockDim.x) ws.row_base[i] = L.row_base[i];
    for (int i = threadIdx.x; i <= A; i += blockDim.x) ws.rec_prefix[i] = L.rec_prefix[i];
}

// Stand-alone layout pass, used when the host wants exact counts before it allocates the
// receive tensors.  Writes aligned per-expert counts and a sequence number to mapped host
// memory; the receive kernel that follows is launched with layout_ready = 1.
__global__ void __launch_bounds__(256, 1) ffn_layout_kernel(const RankCtx c, const FfnWs ws, const ReceiveArgs r) {
    __shared__ LayoutSmem L;
    const Geometry& g = c.g;
    const unsigned ep = ptx::ld_acquire_gpu(&ws.epoch[0]) + 1u;
    const WaitCtx wc{c.status, c.poison, c.budget, c.rank, /*kernel=*/2};
    if (r.tile_cnt != nullptr)
        for (int i = threadIdx.x; i < r.tile_cnt_n; i += blockDim.x) r.tile_cnt[i] = 0u;
    const bool ok = compute_layout(c, wc, ep, L);
    if (ok) publish_layout(c, ws, r, L);
    __syncthreads();
    if (r.write_host_counts) {
        volatile int* hc = ws.host_counts;
        for (int el = threadIdx.x; el < g.experts_local; el += blockDim.x)
            hc[el] = ok ? align_up_dev(L.tot[el], g.alignment) : 0;
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned seq = ws.epoch[2] + 1u;
            ws.epoch[2] = seq;
            hc[g.experts_local] = ok ? (int)seq : -(int)seq;
            __threadfence_system();
        }
    }
}

// NB record buffers per warp: while record i is being scattered to its expert rows, record
// i+1 is already being pulled into the next buffer if its arrival flag is up.
template <int NB>
__global__ void __launch_bounds__(kMaxWarps * 32, 1)
receive_kernel(const RankCtx c, const FfnWs ws, const ReceiveArgs r) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ LayoutSmem L;
    const Geometry& g = c.g;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, NW = blockDim.x >> 5;
    const int G = gridDim.x, cta = blockIdx.x;
    const int A = g.attn, K = g.top_k, EL = g.experts_local, C = g.capacity;
    const int fi = c.role_rank;
    const unsigned ep = ptx::ld_acquire_gpu(&ws.epoch[0]) + 1u;
    const WaitCtx wc{c.status, c.poison, c.budget, c.rank, /*kernel=*/3};
    unsigned char* heap = reinterpret_cast<unsigned char*>(c.peer[c.rank]);
    trace_stamp(c.trace, kTraceReceive, 0);

    bool ok = true;
    if (r.layout_ready) {
        load_layout(c, ws, L);
    } else {
        ok = compute_layout(c, wc, ep, L);
        if (ok && cta == 0) publish_layout(c, ws, r, L);
    }
    trace_stamp(c.trace, kTraceReceive, 1);

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    unsigned char* bufs = smem + kBarBytes + (size_t)warp * NB * g.rec_bytes;
    if (lane == 0) {
        for (int b = 0; b < NB; ++b) ptx::mbar_init(&bars[warp * NB + b], 1);
        ptx::fence_mbar_init();
    }
    __syncwarp();

    const uint32_t* slot_flag = reinterpret_cast<const uint32_t*>(heap + g.f_slot_flag);
    const unsigned char* stage = heap + g.f_stage;
    const int used = g.meta_off + g.meta_bytes;     // bytes of a record that carry data
    const int total = ok ? L.rec_prefix[A] : 0;
    const int sg = g.fp8 ? g.scale_groups : 0;
    unsigned char* rx = static_cast<unsigned char*>(r.recv_x);
    // Work item j of the striped order goes to CTA j % G first and to the next warp only after
    // every CTA has one: a decode-sized exchange then uses every SM's copy engine for one
    // record instead of filling a few SMs with kMaxWarps records each.
    const int first = warp * G + cta, stride = G * NW;
    const int n_w = first < total ? (total - first + stride - 1) / stride : 0;

    auto locate = [&](int i, int& a, int& slot) { locate_striped(L, A, first + i * stride, a, slot); };
    // Start pulling record i into its ring buffer.  Non-blocking mode gives up at once when the
    // record has not arrived; blocking mode spins (bounded).  Returns 1 issued, 0 not yet, -1 dead.
    auto issue = [&](int i, bool blocking) -> int {
        int a, slot;
        locate(i, a, slot);
        int state = 1;
        if (lane == 0) {
            const uint32_t* flag = slot_flag + (size_t)a * C + slot;
            uint32_t seen = ptx::ld_acquire_sys(flag);
            if (seen != ep) {
                if (!blocking) {
                    state = 0;
                } else {
                    const bool arrived = spin_until(wc, [&] {
                        seen = ptx::ld_acquire_sys(flag);
                        return seen == ep;
                    });
                    if (!arrived) {
                        report(wc, kTimeoutRecord, g.ffn + a, ep, ep, seen, slot, total);
                        poison(wc);
                        state = -1;
                    }
                }
            }
            if (state == 1) {
                if (i == 0) trace_stamp(c.trace, kTraceReceiveFirst, 0);
                uint64_t* bar = &bars[warp * NB + (i % NB)];
                ptx::fence_proxy_async_global();
                ptx::mbar_expect_tx(bar, used);
                ptx::bulk_load(bufs + (size_t)(i % NB) * g.rec_bytes, stage + ((size_t)a * C + slot) * g.rec_bytes, used, bar);
            }
        }
        return __shfl_sync(ptx::kFullMask, state, 0);
    };

    int have = 0;       // 1 when record i's load has been issued ahead of time
    for (int i = 0; i < n_w; ++i) {
        if (!have && issue(i, true) < 0) break;
        have = 0;
        if (i + 1 < n_w) {
            // Buffer (i+1) % NB was last read by the stores of record i+1-NB.
            if (lane == 0) ptx::bulk_wait_read<NB - 2>();
            __syncwarp();
            const int st = issue(i + 1, false);
            if (st < 0) break;
            have = st;
        }
        const int b = i % NB;
        const unsigned parity = (i / NB) & 1u;
        unsigned char* buf = bufs + (size_t)b * g.rec_bytes;
        uint64_t* bar = &bars[warp * NB + b];
        bool landed = spin_until(wc, [&] { return ptx::mbar_try_wait(bar, parity); });
        landed = __all_sync(ptx::kFullMask, landed);
        if (!landed) break;
        if (i == 0) trace_stamp(c.trace, kTraceReceiveFirst, 1);
        int a, slot;
        locate(i, a, slot);

        const int* meta = reinterpret_cast<const int*>(buf + g.meta_off);
        int row = -1;
        float w = 0.f;
        if (lane < K) {
            const int e = meta[lane];
            const int el = e - fi * EL;
            if (e >= 0 && el >= 0 && el < EL) {
                row = L.row_base[a * EL + el] + meta[K + lane];
                w = reinterpret_cast<const float*>(meta)[2 * K + lane];
                if (row < 0 || row >= r.rows_cap) {
                    report(wc, kBadIndex, g.ffn + a, ep, r.rows_cap, row, slot, 3);
                    row = -1;
                }
            }
        }
        const int src_token = meta[3 * K];
        const unsigned hits = __ballot_sync(ptx::kFullMask, row >= 0);
        for (unsigned m = hits; m; m &= m - 1) {
            const int k = __ffs(m) - 1;
            const int rk = __shfl_sync(ptx::kFullMask, row, k);
            if (lane == 0) ptx::bulk_store(rx + (size_t)rk * g.payload_bytes, buf, g.payload_bytes);
            const float* sc = reinterpret_cast<const float*>(buf + g.payload_bytes);
            for (int gi = lane; gi < sg; gi += 32) r.recv_scale[(size_t)rk * r.rs0 + (size_t)gi * r.rs1] = sc[gi];
        }
        if (lane == 0) ptx::bulk_commit();
        if (i == 0) trace_stamp(c.trace, kTraceReceiveFirst, 2);
        if (row >= 0) {
            r.recv_w[row] = w;
            r.recv_src[2 * (size_t)row] = a;
            r.recv_src[2 * (size_t)row + 1] = src_token;
        }
        __syncwarp();
    }
    if (lane == 0) ptx::bulk_wait<0>();
    if (n_w > 0) trace_stamp(c.trace, kTraceReceiveFirst, 3);

    __syncthreads();
    trace_stamp(c.trace, kTraceReceive, 2);
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(&ws.ticket[0], 1u) == (unsigned)(G - 1)) {
            ws.ticket[0] = 0;
            ws.epoch[0] = ep;
            __threadfence();
        }
    }
}

// acc[0..8) += the eight BF16 values of v, as exact fp32 additions.  A BF16 is the upper half
// of an fp32, so unpacking is a shift and a mask, and sm_100's packed add does two lanes at once.
__device__ __forceinline__ void acc_bf16x8(float* acc, const uint4& v) {
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 x = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
        const float2 r = __fadd2_rn(make_float2(acc[2 * i], acc[2 * i + 1]), x);
        acc[2 * i] = r.x;
        acc[2 * i + 1] = r.y;
    }
}
__device__ __forceinline__ uint4 pack_bf16x8(const float* acc) {
    uint4 v;
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    return v;
}

constexpr unsigned kReplyFlagPatience = 8;   // polls the flag warp holds back a fence for stragglers
constexpr int kReplyWarps = 8;   // seven reducing warps (16 loads per lane in flight) and one flag warp

__global__ void __launch_bounds__(kReplyWarps * 32, 2)
reply_kernel(const RankCtx c, const FfnWs ws, const unsigned char* __restrict__ rows, int rows_cap) {
    __shared__ LayoutSmem L;
    __shared__ int s_rows[kReplyWarps][kMaxTopK];
    __shared__ int s_done[32];
    const Geometry& g = c.g;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int ND = kReplyWarps - 1;
    const int G = gridDim.x, cta = blockIdx.x;
    const int A = g.attn, K = g.top_k, EL = g.experts_local, C = g.capacity;
    const int fi = c.role_rank;
    const unsigned ep = ptx::ld_acquire_gpu(&ws.epoch[1]) + 1u;
    const WaitCtx wc{c.status, c.poison, c.budget, c.rank, /*kernel=*/4};
    unsigned char* heap = reinterpret_cast<unsigned char*>(c.peer[c.rank]);
    if (tid < 32) s_done[tid] = 0;
    trace_stamp(c.trace, kTraceReply, 0);
    load_layout(c, ws, L);
    const bool dead = poisoned(wc);   // an abandoned receive leaves no layout to reply to

    const unsigned char* stage = heap + g.f_stage;
    unsigned char* reply = heap + g.f_reply;
    const int total = dead ? 0 : L.rec_prefix[A];
    const int nvec = g.hidden / 8;    // 16-byte vectors per row
    auto locate = [&](int item, int& a, int& slot) { locate_striped(L, A, item, a, slot); };

    // Two ways to spread records over the reducing warps, chosen from the live record count:
    //   many records: one warp per record (best throughput, a warp streams a whole row);
    //   few records:  the CTA's warps split one record's columns in chunks of 64 vectors, so a
    //                 decode-sized exchange finishes in a few microseconds instead of a row time.
    constexpr int U = 2, R = 8;
    const int nchunks = (nvec + 32 * U - 1) / (32 * U);
    const bool coop = total * 2 < G * ND;
    const int first = coop ? cta : cta * ND + warp;
    const int stride = coop ? G : G * ND;
    auto count_from = [&](int f0) { return f0 < total ? (total - f0 + stride - 1) / stride : 0; };
    if (warp < ND) {
        const int n_w = count_from(first);
        const int ch0 = coop ? warp : 0, chs = coop ? ND : 1;
        // The routing words of the next record are fetched while the current one is reduced.
        auto fetch = [&](int i, int& a, int& slot, int& e, int& pos) {
            locate(first + i * stride, a, slot);
            const int* meta = reinterpret_cast<const int*>(stage + ((size_t)a * C + slot) * g.rec_bytes + g.meta_off);
            e = -1;
            pos = 0;
            if (lane < K) {
                e = __ldcg(meta + lane);
                pos = __ldcg(meta + K + lane);
            }
        };
        int a_n = 0, slot_n = 0, e_n = -1, pos_n = 0;
        if (n_w > 0) fetch(0, a_n, slot_n, e_n, pos_n);
        for (int i = 0; i < n_w; ++i) {
            const int a = a_n, slot = slot_n, e = e_n, pos = pos_n;
            if (i + 1 < n_w) fetch(i + 1, a_n, slot_n, e_n, pos_n);
            int row = -1;
            {
                const int el = e - fi * EL;
                if (e >= 0 && el >= 0 && el < EL) {
                    row = L.row_base[a * EL + el] + pos;
                    if (row < 0 || row >= rows_cap) row = -1;
                }
            }
            const unsigned hits = __ballot_sync(ptx::kFullMask, row >= 0);
            const int nh = __popc(hits);
            if (row >= 0) s_rows[warp][__popc(hits & ptx::lanemask_lt())] = row;
            __syncwarp();
            unsigned char* out = reply + ((size_t)a * C + slot) * g.row_bytes;
            for (int ch = ch0; ch < nchunks; ch += chs) {
                const int v = ch * 32 * U + lane;
                if (nh == 1) {
                    const unsigned char* src = rows + (size_t)s_rows[warp][0] * g.row_bytes;
                    uint4 x[U];
#pragma unroll
                    for (int u = 0; u < U; ++u)
                        if (v + u * 32 < nvec) x[u] = *reinterpret_cast<const uint4*>(src + (size_t)(v + u * 32) * 16);
#pragma unroll
                    for (int u = 0; u < U; ++u)
                        if (v + u * 32 < nvec) *reinterpret_cast<uint4*>(out + (size_t)(v + u * 32) * 16) = x[u];
                } else {
                    // Rows are fetched eight at a time for two vectors per lane: sixteen 16-byte loads
                    // in flight per lane; the additions still happen in top-k order.
                    float acc[U][8];
#pragma unroll
                    for (int u = 0; u < U; ++u)
#pragma unroll
                        for (int q = 0; q < 8; ++q) acc[u][q] = 0.f;
                    for (int h0 = 0; h0 < nh; h0 += R) {
                        uint4 x[R][U];
#pragma unroll
                        for (int j = 0; j < R; ++j) {
                            if (h0 + j < nh) {
                                const unsigned char* src = rows + (size_t)s_rows[warp][h0 + j] * g.row_bytes;
#pragma unroll
                                for (int u = 0; u < U; ++u)
                                    if (v + u * 32 < nvec) x[j][u] = *reinterpret_cast<const uint4*>(src + (size_t)(v + u * 32) * 16);
                            }
                        }
#pragma unroll
                        for (int j = 0; j < R; ++j) {
                            if (h0 + j < nh) {
#pragma unroll
                                for (int u = 0; u < U; ++u)
                                    if (v + u * 32 < nvec) acc_bf16x8(acc[u], x[j][u]);
                            }
                        }
                    }
#pragma unroll
                    for (int u = 0; u < U; ++u)
                        if (v + u * 32 < nvec)
                            *reinterpret_cast<uint4*>(out + (size_t)(v + u * 32) * 16) = pack_bf16x8(acc[u]);
                }
            }
            __syncwarp();      // every lane's stores are ordered before the hand-off below
            if (lane == 0) ptx::st_release_cta_shared(&s_done[warp], i + 1);
        }
    } else {
        // Flag warp: one system-scope fence covers every record handed over since the last one,
        // so the fence never stalls a reducing warp.  Cooperative mode: a record is complete when
        // every warp has handed it over, lanes share the flags; otherwise lane w follows warp w.
        const int mine = coop ? count_from(cta) : ((lane < ND) ? count_from(cta * ND + lane) : 0);
        int flagged = 0;
        unsigned idle = 0, patience = 0;
        const long long t_begin = clock64();
        while (true) {
            int d = (lane < ND) ? ptx::ld_acquire_cta_shared(&s_done[lane]) : (coop ? mine : 0);
            if (coop) d = __reduce_min_sync(ptx::kFullMask, d);
            // A fence costs microseconds while stores are in flight: hold it back (briefly) until
            // every reducing warp that still owes flags has handed something over.
            const unsigned fresh = __ballot_sync(ptx::kFullMask, d > flagged);
            const unsigned owing = __ballot_sync(ptx::kFullMask, flagged < mine);
            if (fresh != 0 && (fresh == owing || ++patience > kReplyFlagPatience)) {
                patience = 0;
                if (d > flagged) {
                    ptx::fence_acq_rel_sys();
                    for (int j = coop ? flagged + lane : flagged; j < d; j += coop ? 32 : 1) {
                        int a, slot;
                        locate((coop ? cta : cta * ND + lane) + j * stride, a, slot);
                        uint32_t* flag = reinterpret_cast<uint32_t*>(c.peer[g.ffn + a] + g.a_reply_flag) + (size_t)fi * C + slot;
                        ptx::st_relaxed_sys(flag, ep);
                    }
                    flagged = d;
                }
                idle = 0;
            }
            if (__all_sync(ptx::kFullMask, flagged >= mine)) break;
            if (++idle > 1) __nanosleep(64);
            if ((idle & 255u) == 0 && (poisoned(wc) || clock64() - t_begin > 4 * c.budget)) break;
        }
    }

    __syncthreads();
    trace_stamp(c.trace, kTraceReply, 2);
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(&ws.ticket[1], 1u) == (unsigned)(G - 1)) {
            ws.ticket[1] = 0;
            ws.epoch[1] = ep;
            __threadfence();
        }
    }
}

}  // namespace

// Static shared memory of the receive kernel, measured once by configure_ffn.
static int g_receive_static = (int)sizeof(LayoutSmem) + 1024;

static int receive_buffers(const Geometry& g, int max_smem) {
    const int avail = max_smem - kBarBytes - g_receive_static;
    return avail / (3 * g.rec_bytes) >= 4 ? 3 : 2;
}

LaunchShape receive_shape(const Geometry& g, int num_sms, int max_smem) {
    LaunchShape s{};
    const int nb = receive_buffers(g, max_smem);
    int avail = max_smem - kBarBytes - g_receive_static;
    int warps = avail / (nb * g.rec_bytes);
    if (warps > kMaxWarps) warps = kMaxWarps;
    if (warps < 1) warps = 1;
    s.ctas = num_sms;
    s.warps = warps;
    s.smem_bytes = kBarBytes + warps * nb * g.rec_bytes;
    return s;
}

LaunchShape reply_shape(const Geometry& g, int num_sms, int max_smem) {
    (void)g;
    (void)max_smem;
    LaunchShape s{};
    s.ctas = 2 * num_sms;
    s.warps = kReplyWarps;
    s.smem_bytes = 0;
    return s;
}

cudaError_t launch_ffn_layout(const RankCtx& c, const FfnWs& ws, const ReceiveArgs& r, cudaStream_t stream) {
    ffn_layout_kernel<<<1, 256, 0, stream>>>(c, ws, r);
    return cudaGetLastError();
}

cudaError_t launch_receive(const RankCtx& c, const FfnWs& ws, const ReceiveArgs& r, LaunchShape s,
                           cudaStream_t stream) {
    // The ring depth is implied by the shape receive_shape chose.
    const int nb = (s.smem_bytes - kBarBytes) / (s.warps * c.g.rec_bytes);
    if (nb >= 3)
        receive_kernel<3><<<s.ctas, s.warps * 32, s.smem_bytes, stream>>>(c, ws, r);
    else
        receive_kernel<2><<<s.ctas, s.warps * 32, s.smem_bytes, stream>>>(c, ws, r);
    return cudaGetLastError();
}

cudaError_t launch_reply(const RankCtx& c, const FfnWs& ws, const void* rows, int rows_cap, LaunchShape s,
                         cudaStream_t stream) {
    reply_kernel<<<s.ctas, s.warps * 32, s.smem_bytes, stream>>>(c, ws, static_cast<const unsigned char*>(rows),
                                                                rows_cap);
    return cudaGetLastError();
}

cudaError_t configure_ffn(int max_smem) {
    cudaFuncAttributes attr;
    cudaError_t e = cudaFuncGetAttributes(&attr, receive_kernel<3>);
    if (e != cudaSuccess) return e;
    g_receive_static = (int)attr.sharedSizeBytes + 128;
    e = cudaFuncSetAttribute(receive_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem - g_receive_static);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(receive_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                max_smem - g_receive_static);
}

}  // namespace afdep
