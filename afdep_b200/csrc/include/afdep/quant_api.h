// Host interface of the row-wise FP8 quantiser (kernels/quant.cu).
#pragma once
#include <cuda_runtime.h>

namespace afdep {

// x: bf16 [rows, K] (K a multiple of 128) -> q: e4m3 [rows, K], scale element (row, g) at
// scale[row * ss0 + g * ss1].  `limit`, if not null, points at a device int: rows at or beyond
// it are skipped (the end of the last expert segment).  `pow2` rounds every scale up to a power
// of two, the form the hardware block-scaled GEMM takes.
cudaError_t launch_quantize_rows(const void* x, void* q, float* scale, int rows, int K, long long ss0, long long ss1,
                                 const int* limit, bool pow2, int ctas, cudaStream_t stream);

}  // namespace afdep
