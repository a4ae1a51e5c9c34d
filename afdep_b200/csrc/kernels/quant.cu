// Row-wise FP8 quantisation: BF16 [rows, K] -> e4m3 [rows, K] with one fp32 scale per row and
// 128 columns (scale = amax / 448), the activation format of the block-scaled expert GEMM.
// One warp per (row, 128-column group): each lane owns four consecutive values, the group's
// amax is a warp reduction, and the four results leave as one 32-bit store.  Used on FFN ranks
// that receive BF16 rows but keep FP8 expert weights; memory-bound by construction.
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "afdep/quant_api.h"

namespace afdep {

namespace {

__global__ void __launch_bounds__(256) quantize_rows_kernel(const __nv_bfloat16* __restrict__ x, unsigned char* __restrict__ q,
                                                            float* __restrict__ scale, int rows, int K, long long ss0, long long ss1,
                                                            const int* __restrict__ limit, int pow2) {
    const int lane = threadIdx.x & 31;
    const int groups = K / 128;
    const long long total = (long long)rows * groups;
    const int live_rows = limit != nullptr ? min(rows, *limit) : rows;     // rows past the last expert segment are padding
    for (long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < total;
         w += (long long)gridDim.x * (blockDim.x >> 5)) {
        const int row = (int)(w / groups), gidx = (int)(w - (long long)row * groups);
        if (row >= live_rows) continue;
        const size_t off = (size_t)row * K + (size_t)gidx * 128 + lane * 4;
        const uint2 raw = *reinterpret_cast<const uint2*>(x + off);
        const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        const float2 a = __bfloat1622float2(p0), b = __bfloat1622float2(p1);
        float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
        float s = fmaxf(amax, 1e-12f) / 448.f;
        if (pow2) {       // round the scale up to a power of two: exact as an exponent byte
            const unsigned bits = __float_as_uint(s);
            unsigned e = (bits >> 23) & 0xffu;
            if (bits & 0x7fffffu) ++e;
            s = __uint_as_float(min(max(e, 1u), 253u) << 23);
        }
        // true divisions: a value that sits on an e4m3 rounding boundary must land on the same side
        // as in the reference quantiser (the kernel is bound by memory, not by these)
        const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a.x / s, a.y / s), __NV_SATFINITE, __NV_E4M3);
        const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(b.x / s, b.y / s), __NV_SATFINITE, __NV_E4M3);
        *reinterpret_cast<uint32_t*>(q + off) = (uint32_t)lo | ((uint32_t)hi << 16);
        if (lane == 0) scale[(size_t)row * ss0 + (size_t)gidx * ss1] = s;
    }
}

}  // namespace

cudaError_t launch_quantize_rows(const void* x, void* q, float* scale, int rows, int K, long long ss0, long long ss1,
                                 const int* limit, bool pow2, int ctas, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    quantize_rows_kernel<<<ctas, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), static_cast<unsigned char*>(q), scale, rows,
                                                   K, ss0, ss1, limit, pow2 ? 1 : 0);
    return cudaGetLastError();
}

}  // namespace afdep
