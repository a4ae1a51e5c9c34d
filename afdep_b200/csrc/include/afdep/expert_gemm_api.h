// Host interface of the expert GEMM that feeds itself (kernels/expert_gemm.cu).
//
// Same product as the grouped GEMM of gemm_api.h -- C[rows, N] = A[rows, K] * W_e[N, K]^T over
// expert-major row segments -- with two additions:
//   * FP8 operands are scaled by the tensor core itself (tcgen05.mma kind::mxf8f6f4.block_scale):
//     the fp32 scales of the block-scaled format (one per row and 128 columns of A, one per
//     128 x 128 block of W) must be exact powers of two, are turned into exponent bytes and
//     written to tensor memory next to the accumulator, and the whole K extent accumulates in
//     tensor memory.  No per-block promotion through registers.
//   * The rows of A can be gathered by index from another matrix, in particular straight from
//     the wire records in the FFN rank's staging region, so the expert-major copy of the received
//     activations is never written.  In the fused form the same launch also turns arrival flags
//     into the row index (what the receive kernel does otherwise) and starts a row tile as soon
//     as all of its records have landed.
// The reference library has no expert GEMM (callers bring their own); its counterpart of
// "consume a record as it lands" is the per-record expansion kernel
// (deep_ep/include/deep_ep/impls/dispatch_copy_epilogue.cuh:61-142).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "kernels.h"
#include "layout.h"

namespace afdep {

struct ExpertGemmArgs {
    int rows;            // rows of the expert-major row space (the receive bound)
    int N, K;            // W_e is [N, K]; N a multiple of 128, K a multiple of 128
    int experts;
    int alignment;       // expert segments start on multiples of this (a multiple of 128)
    const int* ends;     // device [experts]: end row of every expert segment
    int mx;              // 1: e4m3 operands with power-of-two fp32 block scales; 0: BF16 operands
    long long budget;    // clock64 ticks any wait inside the kernel may take

    // A operand, dense form: the tensor map passed to the launch covers A[rows, K].
    // A operand, gathered form: row r of the row space is the first K elements of
    //   a_rows + row_rec[r] * a_pitch          (row_rec[r] < 0: a row of zeros)
    const unsigned char* a_rows;
    long long a_pitch;
    const int* row_rec;

    // Scales (mx only).  Dense: element (row, kb) at a_scale[row * s0 + kb * s1].  Gathered: K/128
    // floats at byte offset a_scale_off inside the gathered row's record.
    // With a_scale_packed the scales are exponent bytes (UE8M0) packed four to a 32-bit word, one word
    // per row and group of four K blocks: a_scale then points at words ([rows, ceil(K / 512)], strides
    // in words), and a gathered record holds ceil(K / 512) words at a_scale_off.  The words go to
    // tensor memory as they are.
    const float* a_scale;
    long long a_scale_s0, a_scale_s1;
    int a_scale_off;
    int a_scale_packed;
    const float* w_scale;    // [experts][N / 128][K / 128]

    // Epilogue.
    __nv_bfloat16* out;      // [rows, ldc] BF16, or null with out_q
    int ldc;                 // N, or N / 2 with swiglu
    int swiglu;              // 1: W rows alternate 32 gate / 32 up; out = silu(gate) * up
    const float* row_scale;  // optional [rows]
    unsigned char* out_q;    // optional (mx, swiglu, N % 256 == 0): e4m3 [rows, ldc] ...
    float* out_q_scale;      // ... with one power-of-two scale per row and 128 output columns
    long long oqs0, oqs1;
    int* error;              // optional host-visible word set to 1 if a bounded wait gave up
};

// The fused receive: index the exchange's records while the GEMM runs.
struct FusedReceive {
    int enabled;
    RankCtx c;
    FfnWs ws;
    int* row_rec;        // [rows_cap] out: record index (source * capacity + slot) of every row
    float* recv_w;       // [rows_cap] out: routing weight of every row
    int* recv_src;       // [rows_cap][2] out: source attention rank, source token
    unsigned* tile_cnt;  // [rows_cap / 128] rows indexed so far per 128-row tile; zero at launch
    int rows_cap;
};

int expert_gemm_smem_bytes(bool fused);
// `gather`: A comes from a_rows / row_rec instead of map_a.  `fr.enabled` needs `gather`, and the
// grid must be co-resident (the launch is cooperative and fails on the host otherwise).
cudaError_t launch_expert_gemm(const CUtensorMap& map_a, const CUtensorMap& map_w, const ExpertGemmArgs& args, bool gather,
                               const FusedReceive& fr, int ctas, cudaStream_t stream);

}  // namespace afdep
