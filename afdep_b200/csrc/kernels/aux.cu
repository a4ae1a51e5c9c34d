// Secondary primitives on the heap's auxiliary region (see aux_api.h for the layout).
//
// All bulk data moves through one pipeline: a single thread per CTA streams 32 KB chunks with the
// copy engine of its SM -- cp.async.bulk global -> shared into a ring of four stages, then
// cp.async.bulk shared -> global (possibly a peer's memory) -- so the load of a chunk overlaps the
// stores of the ones before it, the SM's other warps stay free, and one chunk can be stored to
// several destinations after a single load.  Every wait is bounded.
#include "afdep/aux_api.h"
#include "afdep/status.cuh"

namespace afdep {

namespace {

constexpr int kThreads = 128;
constexpr int kChunk = 32768;
constexpr int kPipeStages = 4;
constexpr int kPipeSmem = kPipeStages * kChunk + 128;

__device__ __forceinline__ unsigned char* aux_base(const RankCtx& c, int rank) { return reinterpret_cast<unsigned char*>(c.peer[rank]) + c.g.aux_off; }
__device__ __forceinline__ uint32_t* aux_signal(const RankCtx& c, int rank, int word) { return reinterpret_cast<uint32_t*>(aux_base(c, rank)) + word; }
__device__ __forceinline__ unsigned char* aux_data(const RankCtx& c, int rank) { return aux_base(c, rank) + kAuxSignalBytes; }

// Copies `bytes` (a multiple of 16, both sides 16-byte aligned) from `src` to each of the `ndst`
// destinations.  Chunks are dealt round-robin over the CTAs of the grid; thread 0 of a CTA runs
// the pipeline.  `smem` is kPipeSmem bytes, 128-byte aligned.  Returns false if a wait ran out
// (only possible with a broken build: every load is local or a plain peer read).
__device__ bool pipe_copy(unsigned char* const* dst, int ndst, const unsigned char* src, size_t bytes, unsigned char* smem,
                          const WaitCtx& wc) {
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPipeStages * kChunk);
    const size_t nchunks = (bytes + kChunk - 1) / kChunk;
    const size_t first = blockIdx.x, stride = gridDim.x;
    const size_t mine = first < nchunks ? (nchunks - first + stride - 1) / stride : 0;
    if (mine == 0) return true;
    for (int s = 0; s < kPipeStages; ++s) ptx::mbar_init(&bars[s], 1);
    ptx::fence_mbar_init();
    auto chunk_off = [&](size_t j) { return (first + j * stride) * (size_t)kChunk; };
    auto chunk_len = [&](size_t j) { return (uint32_t)min((size_t)kChunk, bytes - chunk_off(j)); };
    auto load = [&](size_t j) {
        const int s = (int)(j % kPipeStages);
        ptx::mbar_expect_tx(&bars[s], chunk_len(j));
        ptx::bulk_load(smem + (size_t)s * kChunk, src + chunk_off(j), chunk_len(j), &bars[s]);
    };
    for (size_t j = 0; j < mine && j < (size_t)(kPipeStages - 1); ++j) load(j);
    bool ok = true;
    for (size_t j = 0; j < mine; ++j) {
        const int s = (int)(j % kPipeStages);
        const unsigned parity = (unsigned)((j / kPipeStages) & 1);
        ok = spin_until(wc, [&] { return ptx::mbar_try_wait(&bars[s], parity); });
        if (!ok) break;
        for (int d = 0; d < ndst; ++d) ptx::bulk_store(dst[d] + chunk_off(j), smem + (size_t)s * kChunk, chunk_len(j));
        ptx::bulk_commit();
        const size_t jn = j + kPipeStages - 1;       // refills the stage chunk j-1 was stored from
        if (jn < mine) {
            ptx::bulk_wait_read<1>();
            load(jn);
        }
    }
    ptx::bulk_wait<0>();                             // every store of this CTA has been performed
    return ok;
}

// True in exactly one thread of the grid: thread 0 of the last CTA to arrive.
__device__ __forceinline__ bool last_cta(unsigned* ticket) {
    __shared__ int s_last;
    __threadfence_system();     // this CTA's stores may target a peer GPU
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned t = atomicAdd(ticket, 1u);
        s_last = (t == gridDim.x - 1);
        if (s_last) *ticket = 0;
    }
    __syncthreads();
    return s_last != 0;
}

// Gather n writes slot [n % 2][rank] of every peer.  A rank can start gather n + 2 (which reuses
// the slots of gather n) only after its own wait of gather n + 1, which needs every peer's push
// of n + 1, which that peer's stream issued after it had copied gather n out of its heap
// (all_gather always hands out a copy): so two slot sets are enough and no acknowledgement is needed.
__global__ void __launch_bounds__(kThreads) allgather_push_kernel(const RankCtx c, const AuxSeq seq, const unsigned char* src,
                                                                  size_t bytes, size_t slot_bytes) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int W = c.g.world;
    const unsigned ep = *reinterpret_cast<volatile unsigned*>(seq.gather) + 1u;
    const WaitCtx wc{c.status, c.poison, c.budget, c.rank, /*kernel=*/9};
    if (threadIdx.x == 0) {
        unsigned char* dst[kMaxRanks];
        for (int p = 0; p < W; ++p) dst[p] = aux_data(c, p) + ((size_t)(ep & 1u) * W + c.rank) * slot_bytes;
        if (!pipe_copy(dst, W, src, bytes, smem, wc)) {
            report(wc, kTimeoutAux, -1, ep, 0, 0, 3, 0);
            poison(wc);
        }
    }
    if (last_cta(seq.ticket + 0) && threadIdx.x < W) {
        ptx::fence_acq_rel_sys();
        ptx::st_relaxed_sys(aux_signal(c, threadIdx.x, c.rank), ep);
    }
}

__global__ void __launch_bounds__(32) allgather_wait_kernel(const RankCtx c, const AuxSeq seq) {
    const int W = c.g.world;
    const unsigned ep = *reinterpret_cast<volatile unsigned*>(seq.gather) + 1u;
    const WaitCtx wc{c.status, c.poison, c.budget, c.rank, /*kernel=*/9};
    if (threadIdx.x < W) {
        uint32_t seen = 0;
        const bool ok = spin_until(wc, [&] {
            seen = ptx::ld_acquire_sys(aux_signal(c, c.rank, threadIdx.x));
            return (int)(seen - ep) >= 0;
        });
        if (!ok) {
            report(wc, kTimeoutAux, threadIdx.x, ep, ep, seen, 0, 0);
            poison(wc);
        }
    }
    __syncwarp();
    if (threadIdx.x == 0) *seq.gather = ep;
}

// After the wait: copy the gathered contributions [world][bytes] out of the heap.  The slot set is
// the parity of the gather count the wait kernel just advanced.
__global__ void __launch_bounds__(256) allgather_copy_out_kernel(const RankCtx c, const AuxSeq seq, unsigned char* out, size_t bytes,
                                                                 size_t slot_bytes) {
    const int W = c.g.world;
    const unsigned ep = *reinterpret_cast<volatile unsigned*>(seq.gather);
    const unsigned char* base = aux_data(c, c.rank) + (size_t)(ep & 1u) * W * slot_bytes;
    const size_t vec = bytes / 16, total = vec * W;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / vec, v = i - r * vec;
        reinterpret_cast<uint4*>(out + r * bytes)[v] = ptx::ld_cg_v4(reinterpret_cast<const uint4*>(base + r * slot_bytes) + v);
    }
}

// Message n from `src` to `dst` travels in slot (n - 1) % inflight of the pair's ring in dst's
// data area.  The sender needs the credit for message n - inflight (dst consumed it), so up to
// `inflight` messages are on their way before a sender ever waits for its receiver.
__global__ void __launch_bounds__(kThreads) p2p_send_kernel(const RankCtx c, const AuxSeq seq, int dst, const unsigned char* src,
                                                            size_t bytes, size_t slot_bytes, int inflight) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_ok;
    const unsigned n = *reinterpret_cast<volatile unsigned*>(seq.sent + dst) + 1u;     // this message's number
    const WaitCtx wc{c.status, c.poison, c.budget, c.rank, /*kernel=*/10};
    if (threadIdx.x == 0) {
        uint32_t seen = 0;
        bool ok = spin_until(wc, [&] {
            seen = ptx::ld_acquire_sys(aux_signal(c, c.rank, 16 + dst));
            return (int)(seen + (unsigned)inflight - n) >= 0;
        });
        if (!ok) {
            report(wc, kTimeoutAux, dst, n, n - (unsigned)inflight, seen, 1, 0);
            poison(wc);
        } else {
            unsigned char* to = aux_data(c, dst) + ((size_t)c.rank * inflight + (n - 1u) % (unsigned)inflight) * slot_bytes;
            ok = pipe_copy(&to, 1, src, bytes, smem, wc);
        }
        s_ok = ok;
    }
    __syncthreads();
    if (last_cta(seq.ticket + 1) && threadIdx.x == 0) {
        if (s_ok) {
            ptx::fence_acq_rel_sys();
            ptx::st_relaxed_sys(aux_signal(c, dst, 8 + c.rank), n);
        }
        seq.sent[dst] = n;
    }
}

__global__ void __launch_bounds__(kThreads) p2p_recv_kernel(const RankCtx c, const AuxSeq seq, int src_rank, unsigned char* dst,
                                                            size_t bytes, size_t slot_bytes, int inflight) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_ok;
    const unsigned n = *reinterpret_cast<volatile unsigned*>(seq.received + src_rank) + 1u;
    const WaitCtx wc{c.status, c.poison, c.budget, c.rank, /*kernel=*/11};
    if (threadIdx.x == 0) {
        uint32_t seen = 0;
        bool ok = spin_until(wc, [&] {
            seen = ptx::ld_acquire_sys(aux_signal(c, c.rank, 8 + src_rank));
            return (int)(seen - n) >= 0;
        });
        if (!ok) {
            report(wc, kTimeoutAux, src_rank, n, n, seen, 2, 0);
            poison(wc);
        } else {
            ptx::fence_proxy_async_global();       // the flag was seen by an ordinary load, the data is read by bulk copies
            const unsigned char* from = aux_data(c, c.rank) + ((size_t)src_rank * inflight + (n - 1u) % (unsigned)inflight) * slot_bytes;
            ok = pipe_copy(&dst, 1, from, bytes, smem, wc);
        }
        s_ok = ok;
    }
    __syncthreads();
    if (last_cta(seq.ticket + 2) && threadIdx.x == 0) {
        if (s_ok) {
            ptx::fence_acq_rel_sys();
            ptx::st_relaxed_sys(aux_signal(c, src_rank, 16 + c.rank), n);     // credit: the slot is free again
        }
        seq.received[src_rank] = n;
    }
}

// Remote row fetch.  One warp per requested row: lane 0 pulls the row from the owning rank's
// shard into shared memory with one bulk load and stores it to the output with one bulk store,
// two rows in flight per warp.  Rows longer than the per-warp buffer fall back to 16-byte loads.
constexpr int kFetchWarps = 8;
constexpr int kFetchRowMax = 8192;

__global__ void __launch_bounds__(kFetchWarps * 32) fetch_rows_kernel(const RankCtx c, const long long* __restrict__ idx, int n,
                                                                       int rows_per_rank, int row_bytes, unsigned char* out) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const WaitCtx wc{c.status, c.poison, c.budget, c.rank, /*kernel=*/13};
    const bool bulk = row_bytes <= kFetchRowMax;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    unsigned char* bufs = smem + 128 + (size_t)warp * 2 * (bulk ? row_bytes : 0);
    if (bulk && lane == 0) {
        ptx::mbar_init(&bars[2 * warp], 1);
        ptx::mbar_init(&bars[2 * warp + 1], 1);
        ptx::fence_mbar_init();
    }
    __syncwarp();
    const int vecs = row_bytes / 16;
    int it = 0;
    bool ok = true;
    for (int i = blockIdx.x * nw + warp; i < n && ok; i += gridDim.x * nw) {
        const long long id = idx[i];
        const long long owner = id / rows_per_rank;
        unsigned char* dst = out + (size_t)i * row_bytes;
        if (id < 0 || owner >= c.g.world) {        // out of range: zero row, never a wild address
            for (int v = lane; v < vecs; v += 32) reinterpret_cast<uint4*>(dst)[v] = make_uint4(0, 0, 0, 0);
            continue;
        }
        const unsigned char* src = aux_data(c, (int)owner) + (size_t)(id - owner * rows_per_rank) * row_bytes;
        if (!bulk) {
            for (int v = lane; v < vecs; v += 32) reinterpret_cast<uint4*>(dst)[v] = ptx::ld_cg_v4(reinterpret_cast<const uint4*>(src) + v);
            continue;
        }
        if (lane == 0) {
            const int b = it & 1;
            if (it >= 2) ptx::bulk_wait_read<1>();           // the store two rows ago has left this buffer
            ptx::mbar_expect_tx(&bars[2 * warp + b], row_bytes);
            ptx::bulk_load(bufs + (size_t)b * row_bytes, src, row_bytes, &bars[2 * warp + b]);
            ok = spin_until(wc, [&] { return ptx::mbar_try_wait(&bars[2 * warp + b], (it >> 1) & 1u); });
            if (ok) {
                ptx::bulk_store(dst, bufs + (size_t)b * row_bytes, row_bytes);
                ptx::bulk_commit();
            } else {
                report(wc, kTimeoutAux, (int)owner, 0, row_bytes, 0, 4, i);
                poison(wc);
            }
        }
        ok = __shfl_sync(ptx::kFullMask, ok, 0);
        ++it;
    }
    if (bulk && lane == 0) ptx::bulk_wait<0>();
}

}  // namespace

cudaError_t configure_aux() {
    cudaError_t e = cudaFuncSetAttribute(allgather_push_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPipeSmem);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(p2p_send_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPipeSmem);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(p2p_recv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPipeSmem);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(fetch_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 + kFetchWarps * 2 * kFetchRowMax);
}

cudaError_t launch_allgather_push(const RankCtx& c, const AuxSeq& seq, const void* src, size_t bytes, size_t slot_bytes,
                                  int ctas, cudaStream_t stream) {
    allgather_push_kernel<<<ctas, kThreads, kPipeSmem, stream>>>(c, seq, static_cast<const unsigned char*>(src), bytes, slot_bytes);
    return cudaGetLastError();
}
cudaError_t launch_allgather_wait(const RankCtx& c, const AuxSeq& seq, cudaStream_t stream) {
    allgather_wait_kernel<<<1, 32, 0, stream>>>(c, seq);
    return cudaGetLastError();
}
cudaError_t launch_allgather_copy_out(const RankCtx& c, const AuxSeq& seq, void* out, size_t bytes, size_t slot_bytes, cudaStream_t stream) {
    if (bytes == 0) return cudaSuccess;
    const size_t total = bytes / 16 * c.g.world;
    const int ctas = (int)((total + 1023) / 1024 < 1 ? 1 : ((total + 1023) / 1024 > 64 ? 64 : (total + 1023) / 1024));
    allgather_copy_out_kernel<<<ctas, 256, 0, stream>>>(c, seq, static_cast<unsigned char*>(out), bytes, slot_bytes);
    return cudaGetLastError();
}
cudaError_t launch_p2p_send(const RankCtx& c, const AuxSeq& seq, int dst, const void* src, size_t bytes, size_t slot_bytes,
                            int inflight, int ctas, cudaStream_t stream) {
    p2p_send_kernel<<<ctas, kThreads, kPipeSmem, stream>>>(c, seq, dst, static_cast<const unsigned char*>(src), bytes, slot_bytes, inflight);
    return cudaGetLastError();
}
cudaError_t launch_p2p_recv(const RankCtx& c, const AuxSeq& seq, int src_rank, void* dst, size_t bytes, size_t slot_bytes,
                            int inflight, int ctas, cudaStream_t stream) {
    p2p_recv_kernel<<<ctas, kThreads, kPipeSmem, stream>>>(c, seq, src_rank, static_cast<unsigned char*>(dst), bytes, slot_bytes, inflight);
    return cudaGetLastError();
}
cudaError_t launch_fetch_rows(const RankCtx& c, const long long* idx, int n, int rows_per_rank, int row_bytes, void* out,
                              int ctas, cudaStream_t stream) {
    const int smem = 128 + (row_bytes <= kFetchRowMax ? kFetchWarps * 2 * row_bytes : 0);
    fetch_rows_kernel<<<ctas, kFetchWarps * 32, smem, stream>>>(c, idx, n, rows_per_rank, row_bytes, static_cast<unsigned char*>(out));
    return cudaGetLastError();
}

}  // namespace afdep
