// Host interface of the grouped expert GEMM (kernels/grouped_gemm.cu).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "layout.h"

namespace afdep {

struct GroupedGemmArgs {
    int rows;            // rows of A / out (the receive bound)
    int N, K;            // W_e is [N, K]; both multiples of 128
    int experts;         // local experts
    int alignment;       // expert segments start on multiples of this (itself a multiple of 128)
    const int* ends;     // device [experts]: end row of each expert segment (recv_count_psum)
    __nv_bfloat16* out;  // [rows, ldc]
    int ldc;             // N, or N / 2 with swiglu
    int swiglu;          // 1: W rows alternate 32 gate / 32 up; out = silu(gate) * up with N/2 columns
    const float* row_scale;   // optional [rows]: routing weight applied to the output row
    int fp8;             // 1: A and W are e4m3 with the scales below
    const float* a_scale;     // element (row, kb) at a_scale[row * s0 + kb * s1]
    long long a_scale_s0, a_scale_s1;
    const float* w_scale;     // [experts][N / 128][K / 128]
    // Optional, FP8 operands with swiglu only: write the SwiGLU output as e4m3 with one fp32
    // scale per row and 128 columns (amax / 448) instead of BF16 `out`, ready to be the A operand
    // of an FP8 down projection.  Needs N to be a multiple of 256.
    unsigned char* out_q;     // [rows, ldc] e4m3
    float* out_q_scale;       // element (row, g) at out_q_scale[row * oqs0 + g * oqs1], g < ldc / 128
    long long oqs0, oqs1;
    int* error;          // optional device word set to 1 if a bounded wait gave up
};

int grouped_gemm_smem_bytes();
cudaError_t launch_grouped_gemm(const CUtensorMap& map_a, const CUtensorMap& map_w, const GroupedGemmArgs& args, int ctas,
                                cudaStream_t stream);
// Host-visible error word of this device's GEMM launches (mapped pinned memory): `device` is the
// pointer kernels write through, `host` the one the runtime polls.  Allocated on first use.
struct GemmErrorWord {
    int* device;
    volatile int* host;
};
GemmErrorWord gemm_error_word(int device_ordinal);

}  // namespace afdep
