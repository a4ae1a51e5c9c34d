// Host interface of the stand-alone routing-layout operation (kernels/layout.cu).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>

namespace afdep {

constexpr int kRouteLayoutWarps = 8;
constexpr int kRouteLayoutMaxCtas = 32;
constexpr int kRouteLayoutHeaderBytes = 64;   // poison words, epoch, ticket

// Bytes of zero-initialised global scratch a launch needs for this geometry.
size_t route_layout_scratch_bytes(int num_experts, int ffn_ranks);
int route_layout_ctas(int tokens);

// ids [T][K] int64; outputs: route_e/route_pos [T][K], tok_slot [T][F], counts [F + E]
// (records per FFN rank, then choices per expert; all -1 if the launch gave up).
cudaError_t launch_route_layout(const long long* ids, int T, int K, int E, int F, void* scratch, int* route_e,
                                int* route_pos, int* tok_slot, int* counts, long long budget, cudaStream_t stream);

}  // namespace afdep
