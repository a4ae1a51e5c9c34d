// Row layout of one exchange on an FFN rank, as every FFN-side kernel keeps it in shared memory:
// where the rows of each (source, expert) pair start, how many records each source sent, and
// the order in which the kernels walk the records.  Shared by the receive and reply kernels and
// by the expert GEMM that gathers its rows straight from the staging records.
#pragma once
#include "kernels.h"
#include "layout.h"

namespace afdep {

struct LayoutSmem {
    int row_base[kMaxRanks * kMaxExpertsLocal];   // [attn][experts_local]
    int tot[kMaxExpertsLocal];
    int start[kMaxExpertsLocal];
    int rec_prefix[kMaxRanks + 1];
    int dead;
};

// Copies the layout the last receive (or the stand-alone layout pass) published.
__device__ __forceinline__ void load_layout(const RankCtx& c, const FfnWs& ws, LayoutSmem& L) {
    const Geometry& g = c.g;
    const int A = g.attn, EL = g.experts_local;
    for (int i = threadIdx.x; i < A * EL; i += blockDim.x) L.row_base[i] = ws.row_base[i];
    for (int i = threadIdx.x; i <= A; i += blockDim.x) L.rec_prefix[i] = ws.rec_prefix[i];
    if (threadIdx.x == 0) L.dead = 0;
    __syncthreads();
}


// Dense work index -> (source, slot), ordered by slot first and source second, so that the
// records of all sources advance together: every attention rank starts seeing its rows (and
// its reply flags) from the beginning of the kernel instead of one source after the other.
__device__ __forceinline__ void locate_striped(const LayoutSmem& L, int A, int j, int& a, int& slot) {
    // cum(s) = number of records with slot < s = sum over sources of min(count, s)
    int lo = 0, hi = 1;
    for (int q = 0; q < A; ++q) hi = max(hi, L.rec_prefix[q + 1] - L.rec_prefix[q]);
    // largest s with cum(s) <= j
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        int cum = 0;
        for (int q = 0; q < A; ++q) cum += min(L.rec_prefix[q + 1] - L.rec_prefix[q], mid);
        if (cum <= j) lo = mid; else hi = mid;
    }
    int cum = 0;
    for (int q = 0; q < A; ++q) cum += min(L.rec_prefix[q + 1] - L.rec_prefix[q], lo);
    int r = j - cum;            // r-th source (in rank order) that still has a record at this slot
    slot = lo;
    a = 0;
    for (int q = 0; q < A; ++q) {
        if (L.rec_prefix[q + 1] - L.rec_prefix[q] > lo) {
            if (r == 0) {
                a = q;
                break;
            }
            --r;
        }
    }
}

}  // namespace afdep
