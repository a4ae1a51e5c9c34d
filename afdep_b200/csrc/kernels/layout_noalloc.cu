// Allocation-free variant of the routing-layout operation; see route_layout_noalloc.h for
// who needs it and the rules of use.  The kernel is the same algorithm as the allocating
// entry point (route_layout.cuh); only the home of the cross-CTA scratch differs: a static
// device array instead of memory the caller provides.
#include <mutex>
#include <string>

#include "afdep/route_layout.cuh"
#include "afdep/route_layout_api.h"
#include "afdep/route_layout_noalloc.h"

namespace {

constexpr int kMaxCols = AFDEP_NOALLOC_MAX_FFN_RANKS + AFDEP_NOALLOC_MAX_EXPERTS;
constexpr size_t kScratchBytes =
    afdep::kRouteLayoutHeaderBytes + (size_t)afdep::kRouteLayoutMaxCtas * kMaxCols * sizeof(unsigned long long);
static_assert(kScratchBytes == AFDEP_NOALLOC_SCRATCH_BYTES, "header and kernel disagree on the scratch size");

// Zero at module load.  In host code this name is only a handle for cudaGetSymbolAddress;
// it is never passed to a kernel as if it were a device pointer.
static __device__ __align__(256) unsigned char g_layout_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
unsigned char* g_scratch_ptr[kMaxDevices] = {};
std::mutex g_setup_mutex;
thread_local std::string t_error;

__global__ void __launch_bounds__(afdep::kRouteLayoutWarps * 32, 1)
route_layout_noalloc_kernel(const long long* __restrict__ ids, int T, int K, int E, int F, unsigned char* scratch,
                            int* route_e, int* route_pos, int* tok_slot, int* counts, long long budget) {
    extern __shared__ __align__(128) unsigned char smem[];
    int* words = reinterpret_cast<int*>(scratch);
    unsigned* epoch = reinterpret_cast<unsigned*>(scratch + 16);
    unsigned* ticket = reinterpret_cast<unsigned*>(scratch + 20);
    unsigned long long* agg = reinterpret_cast<unsigned long long*>(scratch + afdep::kRouteLayoutHeaderBytes);
    const unsigned ep = afdep::ptx::ld_acquire_gpu(epoch) + 1u;
    const afdep::WaitCtx wc{nullptr, words, budget, 0, /*kernel=*/8};
    const int ncols = F + E;
    afdep::RouteLayoutJob job;
    job.ids = ids;
    job.T = T;
    job.K = K;
    job.E = E;
    job.EL = E / F;
    job.F = F;
    job.ep = ep;
    job.agg = agg;
    job.out = afdep::RouteLayoutOut{route_e, route_pos, tok_slot};
    job.wh = reinterpret_cast<int*>(smem);
    job.tot = job.wh + (blockDim.x >> 5) * ncols;
    job.lb = job.tot + ncols;
    job.local = nullptr;
    job.redundant = 0;
    job.trace = nullptr;
    int* tot = job.tot;
    int* lb = job.lb;
    const bool ok = afdep::route_layout_phase(job, wc);
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

int fail(int code, const std::string& text) {
    t_error = text;
    return code;
}

// Device address of the static scratch on the current device, looked up once per device.
int scratch_for_current_device(unsigned char** out, long long* budget) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(AFDEP_NOALLOC_CUDA_ERROR, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(AFDEP_NOALLOC_BAD_ARGUMENT, "device ordinal out of range");
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_layout_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return fail(AFDEP_NOALLOC_CUDA_ERROR, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
        g_scratch_ptr[dev] = static_cast<unsigned char*>(ptr);
    }
    int khz = 0;
    e = cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev);
    if (e != cudaSuccess) return fail(AFDEP_NOALLOC_CUDA_ERROR, std::string("cudaDeviceGetAttribute: ") + cudaGetErrorString(e));
    *out = g_scratch_ptr[dev];
    *budget = (long long)khz * 1000ll * 5ll;   // five seconds of SM clock for the look-back wait
    return AFDEP_NOALLOC_OK;
}

}  // namespace

extern "C" int afdep_route_layout_noalloc(const long long* ids, int tokens, int top_k, int num_experts, int ffn_ranks,
                                          int* route_e, int* route_pos, int* tok_slot, int* counts, void* stream) {
    if (tokens < 0 || top_k < 1 || num_experts < 1 || ffn_ranks < 1 || num_experts % ffn_ranks != 0)
        return fail(AFDEP_NOALLOC_BAD_ARGUMENT, "tokens >= 0, top_k >= 1 and num_experts a positive multiple of ffn_ranks are required");
    if (num_experts > AFDEP_NOALLOC_MAX_EXPERTS || ffn_ranks > AFDEP_NOALLOC_MAX_FFN_RANKS || top_k > AFDEP_NOALLOC_MAX_TOP_K)
        return fail(AFDEP_NOALLOC_TOO_LARGE,
                    "the built-in scratch holds at most 256 experts over 8 FFN ranks with top_k <= 32; got " +
                        std::to_string(num_experts) + " experts, " + std::to_string(ffn_ranks) + " ranks, top_k " +
                        std::to_string(top_k) + " (use route_layout with caller-provided scratch instead)");
    if (counts == nullptr || (tokens > 0 && (ids == nullptr || route_e == nullptr || route_pos == nullptr || tok_slot == nullptr)))
        return fail(AFDEP_NOALLOC_BAD_ARGUMENT, "null input or output pointer");
    unsigned char* scratch = nullptr;
    long long budget = 0;
    const int rc = scratch_for_current_device(&scratch, &budget);
    if (rc != AFDEP_NOALLOC_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // The array keeps the previous call's contents.  Aggregates are epoch-tagged and need no
    // reset; the error words must start at zero.
    cudaError_t e = cudaMemsetAsync(scratch, 0, 16, s);
    if (e != cudaSuccess) return fail(AFDEP_NOALLOC_CUDA_ERROR, std::string("cudaMemsetAsync: ") + cudaGetErrorString(e));
    const int smem = afdep::route_layout_scratch_ints(afdep::kRouteLayoutWarps, ffn_ranks + num_experts) * 4;
    route_layout_noalloc_kernel<<<afdep::route_layout_ctas(tokens), afdep::kRouteLayoutWarps * 32, smem, s>>>(
        ids, tokens, top_k, num_experts, ffn_ranks, scratch, route_e, route_pos, tok_slot, counts, budget);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(AFDEP_NOALLOC_CUDA_ERROR, std::string("kernel launch: ") + cudaGetErrorString(e));
    return AFDEP_NOALLOC_OK;
}

extern "C" const char* afdep_route_layout_noalloc_error(void) { return t_error.c_str(); }
