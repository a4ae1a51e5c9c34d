// Bounded device-side waiting and error reporting.  Every spin in this library goes through
// `spin_until`: it gives up after a clock budget or as soon as another wait of the same
// launch has given up, records the reason once in the host-visible Status block, and lets
// the kernel run to its normal end.  The reference instead prints and traps
// (deep_ep/include/deep_ep/common/comm.cuh:30-54), which kills the CUDA context.
#pragma once
#include "layout.h"
#include "ptx.cuh"

namespace afdep {

// Device words behind RankCtx::poison.
enum DevWord : int {
    kPoison = 0,      // non-zero once any wait of this Buffer has been abandoned
    kClaim = 1,       // first error code; decides which thread fills in the Status block
    kBadRoutes = 2,   // illegal routes seen since the status was last cleared
};

struct WaitCtx {
    Status* status;          // mapped host memory, written by the claiming thread only
    int* poison;             // device words, see DevWord
    long long budget;        // clock64 ticks
    int rank;
    int kernel;
};

__device__ __forceinline__ void report(const WaitCtx& w, int code, int peer, unsigned epoch, long long expected,
                                       long long observed, int d0 = 0, int d1 = 0) {
    if (atomicCAS(&w.poison[kClaim], 0, code) == 0 && w.status != nullptr) {
        volatile Status* s = w.status;
        s->kernel = w.kernel;
        s->rank = w.rank;
        s->peer = peer;
        s->epoch = epoch;
        s->expected = expected;
        s->observed = observed;
        s->detail0 = d0;
        s->detail1 = d1;
        __threadfence_system();
        s->code = code;   // written last: the host treats a non-zero code as a complete record
        __threadfence_system();
    }
}

// Returns true when `ready()` became true, false when the wait was abandoned.
template <class Ready>
__device__ __forceinline__ bool spin_until(const WaitCtx& w, Ready ready) {
    if (ready()) return true;
    const long long t0 = clock64();
    unsigned it = 0;
    while (true) {
        if (ready()) return true;
        if ((++it & 31u) == 0) {
            if (*(volatile int*)(w.poison + kPoison) != 0) return false;
            if (clock64() - t0 > w.budget) return false;
        }
    }
}

// One thread per CTA records a time stamp when tracing is on.
__device__ __forceinline__ void trace_stamp(unsigned long long* trace, int kernel, int stamp) {
    if (trace != nullptr && threadIdx.x == 0 && blockIdx.x < 320)
        trace[((size_t)kernel * 320 + blockIdx.x) * 4 + stamp] = ptx::globaltimer_ns();
}

// The same from whichever single thread the caller picked.
__device__ __forceinline__ void trace_stamp_here(unsigned long long* trace, int kernel, int stamp) {
    if (trace != nullptr && blockIdx.x < 320) trace[((size_t)kernel * 320 + blockIdx.x) * 4 + stamp] = ptx::globaltimer_ns();
}

__device__ __forceinline__ void poison(const WaitCtx& w) { atomicExch(w.poison + kPoison, 1); }
__device__ __forceinline__ bool poisoned(const WaitCtx& w) { return *(volatile int*)(w.poison + kPoison) != 0; }

}  // namespace afdep
