// Secondary primitives on the heap's auxiliary region (see aux_api.h for the layout).
#include "afdep/aux_api.h"
#include "afdep/status.cuh"

namespace afdep {

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ unsigned char* aux_base(const RankCtx& c, int rank) { return reinterpret_cast<unsigned char*>(c.peer[rank]) + c.g.aux_off; }
__device__ __forceinline__ uint32_t* aux_signal(const RankCtx& c, int rank, int word) { return reinterpret_cast<uint32_t*>(aux_base(c, rank)) + word; }
__device__ __forceinline__ unsigned char* aux_data(const RankCtx& c, int rank) { return aux_base(c, rank) + kAuxSignalBytes; }

// Grid-strided 16-byte copy (sizes are multiples of 16, pointers 16-byte aligned).
__device__ __forceinline__ void copy16(unsigned char* dst, const unsigned char* src, size_t bytes) {
    const size_t n = bytes / 16;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
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

__global__ void __launch_bounds__(kThreads) allgather_push_kernel(const RankCtx c, const AuxSeq seq, const unsigned char* src,
                                                                  size_t bytes, size_t slot_bytes) {
    const int W = c.g.world;
    const unsigned ep = *reinterpret_cast<volatile unsigned*>(seq.gather) + 1u;
    for (int p = 0; p < W; ++p) copy16(aux_data(c, p) + (size_t)c.rank * slot_bytes, src, bytes);
    if (last_cta(seq.ticket) && threadIdx.x < W) {
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

__global__ void __launch_bounds__(kThreads) p2p_send_kernel(const RankCtx c, const AuxSeq seq, int dst, const unsigned char* src,
                                                            size_t bytes, size_t slot_bytes) {
    __shared__ int s_ok;
    const unsigned n = *reinterpret_cast<volatile unsigned*>(seq.sent + dst) + 1u;     // this message's number
    const WaitCtx wc{c.status, c.poison, c.budget, c.rank, /*kernel=*/10};
    if (threadIdx.x == 0) {
        // one slot per (source, destination) pair: the previous message must have been consumed
        uint32_t seen = 0;
        const bool ok = spin_until(wc, [&] {
            seen = ptx::ld_acquire_sys(aux_signal(c, c.rank, 16 + dst));
            return (int)(seen - (n - 1u)) >= 0;
        });
        if (!ok) {
            report(wc, kTimeoutAux, dst, n, n - 1u, seen, 1, 0);
            poison(wc);
        }
        s_ok = ok;
    }
    __syncthreads();
    if (s_ok) copy16(aux_data(c, dst) + (size_t)c.rank * slot_bytes, src, bytes);
    if (last_cta(seq.ticket) && threadIdx.x == 0) {
        if (s_ok) {
            ptx::fence_acq_rel_sys();
            ptx::st_relaxed_sys(aux_signal(c, dst, 8 + c.rank), n);
        }
        seq.sent[dst] = n;
    }
}

__global__ void __launch_bounds__(kThreads) p2p_recv_kernel(const RankCtx c, const AuxSeq seq, int src_rank, unsigned char* dst,
                                                            size_t bytes, size_t slot_bytes) {
    __shared__ int s_ok;
    const unsigned n = *reinterpret_cast<volatile unsigned*>(seq.received + src_rank) + 1u;
    const WaitCtx wc{c.status, c.poison, c.budget, c.rank, /*kernel=*/11};
    if (threadIdx.x == 0) {
        uint32_t seen = 0;
        const bool ok = spin_until(wc, [&] {
            seen = ptx::ld_acquire_sys(aux_signal(c, c.rank, 8 + src_rank));
            return (int)(seen - n) >= 0;
        });
        if (!ok) {
            report(wc, kTimeoutAux, src_rank, n, n, seen, 2, 0);
            poison(wc);
        }
        s_ok = ok;
    }
    __syncthreads();
    if (s_ok) copy16(dst, aux_data(c, c.rank) + (size_t)src_rank * slot_bytes, bytes);
    if (last_cta(seq.ticket) && threadIdx.x == 0) {
        if (s_ok) {
            ptx::fence_acq_rel_sys();
            ptx::st_relaxed_sys(aux_signal(c, src_rank, 16 + c.rank), n);     // credit: the slot is free again
        }
        seq.received[src_rank] = n;
    }
}

// One warp per requested row: 16-byte loads straight from the owning rank's shard.
__global__ void __launch_bounds__(kThreads) fetch_rows_kernel(const RankCtx c, const long long* __restrict__ idx, int n,
                                                              int rows_per_rank, int row_bytes, unsigned char* out) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int vecs = row_bytes / 16;
    for (int i = blockIdx.x * nw + warp; i < n; i += gridDim.x * nw) {
        const long long id = idx[i];
        const long long owner = id / rows_per_rank;
        uint4* dst = reinterpret_cast<uint4*>(out + (size_t)i * row_bytes);
        if (id < 0 || owner >= c.g.world) {        // out of range: zero row, never a wild address
            for (int v = lane; v < vecs; v += 32) dst[v] = make_uint4(0, 0, 0, 0);
            continue;
        }
        const uint4* src = reinterpret_cast<const uint4*>(aux_data(c, (int)owner) + (size_t)(id - owner * rows_per_rank) * row_bytes);
        for (int v = lane; v < vecs; v += 32) dst[v] = ptx::ld_cg_v4(src + v);
    }
}

}  // namespace

cudaError_t launch_allgather_push(const RankCtx& c, const AuxSeq& seq, const void* src, size_t bytes, size_t slot_bytes,
                                  int ctas, cudaStream_t stream) {
    allgather_push_kernel<<<ctas, kThreads, 0, stream>>>(c, seq, static_cast<const unsigned char*>(src), bytes, slot_bytes);
    return cudaGetLastError();
}
cudaError_t launch_allgather_wait(const RankCtx& c, const AuxSeq& seq, cudaStream_t stream) {
    allgather_wait_kernel<<<1, 32, 0, stream>>>(c, seq);
    return cudaGetLastError();
}
cudaError_t launch_p2p_send(const RankCtx& c, const AuxSeq& seq, int dst, const void* src, size_t bytes, size_t slot_bytes,
                            int ctas, cudaStream_t stream) {
    p2p_send_kernel<<<ctas, kThreads, 0, stream>>>(c, seq, dst, static_cast<const unsigned char*>(src), bytes, slot_bytes);
    return cudaGetLastError();
}
cudaError_t launch_p2p_recv(const RankCtx& c, const AuxSeq& seq, int src_rank, void* dst, size_t bytes, size_t slot_bytes,
                            int ctas, cudaStream_t stream) {
    p2p_recv_kernel<<<ctas, kThreads, 0, stream>>>(c, seq, src_rank, static_cast<unsigned char*>(dst), bytes, slot_bytes);
    return cudaGetLastError();
}
cudaError_t launch_fetch_rows(const RankCtx& c, const long long* idx, int n, int rows_per_rank, int row_bytes, void* out,
                              int ctas, cudaStream_t stream) {
    fetch_rows_kernel<<<ctas, kThreads, 0, stream>>>(c, idx, n, rows_per_rank, row_bytes, static_cast<unsigned char*>(out));
    return cudaGetLastError();
}

}  // namespace afdep
