// Stand-alone routing layout: the first phase of dispatch as an operation of its own.
//
// Given the [T, K] expert ids of one source it returns, deterministically, the cleaned ids,
// the position of every choice among the source's choices of the same expert, the record
// slot of every (token, FFN rank) pair and the per-rank / per-expert totals — everything a
// caller needs to pre-plan an exchange, size expert batches or test routing code.  The grid
// cooperates through a small global scratch area (epoch word, finish ticket and one
// epoch-tagged aggregate row per CTA); see route_layout.cuh for the algorithm.
#include "afdep/kernels.h"
#include "afdep/route_layout.cuh"
#include "afdep/route_layout_api.h"

namespace afdep {

namespace {

__global__ void __launch_bounds__(kRouteLayoutWarps * 32, 1)
route_layout_kernel(const long long* __restrict__ ids, int T, int K, int E, int F, unsigned char* scratch, int* route_e,
                    int* route_pos, int* tok_slot, int* counts, long long budget) {
    extern __shared__ __align__(128) unsigned char smem[];
    int* words = reinterpret_cast<int*>(scratch);                    // [0..3] poison words
    unsigned* epoch = reinterpret_cast<unsigned*>(scratch + 16);
    unsigned* ticket = reinterpret_cast<unsigned*>(scratch + 20);
    unsigned long long* agg = reinterpret_cast<unsigned long long*>(scratch + kRouteLayoutHeaderBytes);
    const unsigned ep = ptx::ld_acquire_gpu(epoch) + 1u;
    const WaitCtx wc{nullptr, words, budget, 0, /*kernel=*/7};
    const int ncols = F + E;
    RouteLayoutJob job;
    job.ids = ids;
    job.T = T;
    job.K = K;
    job.E = E;
    job.EL = E / F;
    job.F = F;
    job.ep = ep;
    job.agg = agg;
    job.out = RouteLayoutOut{route_e, route_pos, tok_slot};
    job.wh = reinterpret_cast<int*>(smem);
    job.tot = job.wh + (blockDim.x >> 5) * ncols;
    job.lb = job.tot + ncols;
    job.local = nullptr;
    job.redundant = 0;
    job.trace = nullptr;
    int* tot = job.tot;
    int* lb = job.lb;
    const bool ok = route_layout_phase(job, wc);
    if (blockIdx.x == gridDim.x - 1) {
        for (int col = threadIdx.x; col < ncols; col += blockDim.x) counts[col] = ok ? lb[col] + tot[col] : -1;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
            *ticket = 0;
            *epoch = ep;
            __threadfence();
        }
    }
}

}  // namespace

size_t route_layout_scratch_bytes(int num_experts, int ffn_ranks) {
    return kRouteLayoutHeaderBytes + (size_t)kRouteLayoutMaxCtas * (ffn_ranks + num_experts) * sizeof(unsigned long long);
}

int route_layout_ctas(int tokens) {
    int ctas = (tokens + kRouteLayoutWarps * 4 - 1) / (kRouteLayoutWarps * 4);
    if (ctas < 1) ctas = 1;
    return ctas < kRouteLayoutMaxCtas ? ctas : kRouteLayoutMaxCtas;
}

cudaError_t launch_route_layout(const long long* ids, int T, int K, int E, int F, void* scratch, int* route_e,
                                int* route_pos, int* tok_slot, int* counts, long long budget, cudaStream_t stream) {
    const int smem = route_layout_scratch_ints(kRouteLayoutWarps, F + E) * 4;
    // per device context, so set on every launch instead of once per process
    cudaError_t e = cudaFuncSetAttribute(route_layout_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e != cudaSuccess) return e;
    route_layout_kernel<<<route_layout_ctas(T), kRouteLayoutWarps * 32, smem, stream>>>(
        ids, T, K, E, F, static_cast<unsigned char*>(scratch), route_e, route_pos, tok_slot, counts, budget);
    return cudaGetLastError();
}

}  // namespace afdep
