// Launch interface between the host runtime and the CUDA translation units.  Plain
// pointers only, so the kernel files never include torch headers.
//
// One exchange is four launches, two per role:
//   attention: launch_dispatch  ...  launch_collect
//   FFN:       launch_receive   ...  launch_reply
// The reference needs the same four entry points on *every* rank plus two global GPU
// barriers around each transport kernel (deep_ep/include/deep_ep/impls/dispatch.cuh,
// combine.cuh); here ranks only ever wait on point-to-point epoch flags.
#pragma once
#include <cuda_runtime.h>

#include "layout.h"

namespace afdep {

struct RankCtx {
    Geometry g;
    int rank;        // global rank, FFN ranks first
    int role_rank;   // index among the ranks of the same role
    char* peer[kMaxRanks];   // heap base of every rank as mapped into this process
    Status* status;  // device pointer to mapped pinned host memory
    int* poison;     // device word
    long long budget;   // clock64 ticks a wait may spin
    int bounds_check;   // verify computed rows/slots before use
    // Optional device buffer [kTraceRows][kTraceCtas][4] of %globaltimer stamps (ns).  Rows
    // dispatch/receive/reply/collect: start, end of the kernel's first phase, end of its main
    // loop, and (dispatch) counts released to the FFN ranks / (receive) counts of all sources seen.  Row layout (inside dispatch): after set-up, after ranking, after the
    // look-back, after the fix-up.  Rows "first": progress of warp 0's first record (receive) or
    // token (collect) in every CTA that has one.  Null when tracing is off.
    unsigned long long* trace;
};

constexpr int kTraceCtas = 320;
enum TraceKernel : int {
    kTraceDispatch = 0, kTraceReceive = 1, kTraceReply = 2, kTraceCollect = 3, kTraceLayout = 4,
    // First record / token of warp 0 in every CTA that has one:
    kTraceReceiveFirst = 5,   // arrival flag seen, record landed in smem, stores committed, stores complete
    kTraceCollectFirst = 6,   // reply flags seen, rows landed in smem, output stored, unused
};
constexpr int kTraceRows = 7;

// Device-local scratch of an attention rank (not visible to peers).
struct AttnWs {
    unsigned* epoch;    // [0] dispatch, [1] collect: exchanges completed so far
    unsigned* ticket;   // [0] dispatch, [1] collect: CTAs that reached the end of the launch
    unsigned long long* agg;   // [max_ctas][ffn + num_experts]: (epoch << 32 | count)
    unsigned* chunk_done;      // [max_ctas]: epoch at which that CTA's chunk of the layout became final
    int* route_e;       // [capacity][top_k] expert or -1
    int* route_pos;     // [capacity][top_k] rank of the choice within (source, expert)
    int* tok_slot;      // [capacity][ffn] record slot on that FFN rank or -1
};

// Device-local scratch of an FFN rank.
struct FfnWs {
    unsigned* epoch;    // [0] receive, [1] reply, [2] host-count sequence
    unsigned* ticket;   // [0] receive, [1] reply
    int* row_base;      // [attn][experts_local] first row of (source, expert)
    int* rec_prefix;    // [attn + 1] prefix sum of records per source
    int* ends;          // [experts_local] copy of the last receive's prefix sums
    int* host_counts;   // mapped pinned host memory: [experts_local] aligned counts, then seq
};

struct DispatchArgs {
    const void* x;          // [T][hidden] bf16 or e4m3, contiguous
    const float* x_scale;   // FP8 only: element (t, g) at x_scale[t * ss0 + g * ss1]
    long long ss0, ss1;
    const long long* ids;   // [T][top_k] int64, or null with ids32
    const int* ids32;       // [T][top_k] int32 (Buffer option topk_idx_bits=32)
    const float* weights;   // [T][top_k]
    int T;
    // 0: arrival flags are released by the CTA's flag warp behind a system-scope fence.
    // 1: experimental, AFDEP_FLAG_MODE=1: the data warp that saw its bulk stores complete
    //    releases the flags itself with relaxed system-scope stores and no fence.
    int flag_mode;
};

struct ReceiveArgs {
    void* recv_x;           // [rows_cap][hidden]
    float* recv_scale;      // FP8 only: element (row, g) at recv_scale[row * rs0 + g * rs1]
    long long rs0, rs1;
    float* recv_w;          // [rows_cap]
    int* recv_src;          // [rows_cap][2]: source attention rank, source token
    int* psum;              // [experts_local] end row of every expert segment
    long long* expert_stats;  // optional [experts_local]: running total of rows received per expert
    int rows_cap;
    int layout_ready;       // 1: launch_ffn_layout already ran for this exchange
    int write_host_counts;  // layout kernel only
    unsigned* tile_cnt;     // layout kernel only, optional: per-tile row counters of the fused expert path, zeroed here
    int tile_cnt_n;
};

struct LaunchShape {
    int ctas;
    int warps;
    int smem_bytes;
};

// Pick warps/smem for a kernel given the CTA budget and the device's opt-in shared memory.
LaunchShape dispatch_shape(const Geometry& g, int tokens, int num_sms, int max_smem);
LaunchShape receive_shape(const Geometry& g, int num_sms, int max_smem);
LaunchShape reply_shape(const Geometry& g, int num_sms, int max_smem);
LaunchShape collect_shape(const Geometry& g, int tokens, int num_sms, int max_smem);
int max_dispatch_ctas();   // rows of AttnWs::agg

cudaError_t launch_dispatch(const RankCtx& c, const AttnWs& ws, const DispatchArgs& a, LaunchShape s,
                            cudaStream_t stream);
cudaError_t launch_collect(const RankCtx& c, const AttnWs& ws, void* out, int T, LaunchShape s,
                           cudaStream_t stream);
cudaError_t launch_ffn_layout(const RankCtx& c, const FfnWs& ws, const ReceiveArgs& r, cudaStream_t stream);
cudaError_t launch_receive(const RankCtx& c, const FfnWs& ws, const ReceiveArgs& r, LaunchShape s,
                           cudaStream_t stream);
cudaError_t launch_reply(const RankCtx& c, const FfnWs& ws, const void* rows, int rows_cap, LaunchShape s,
                         cudaStream_t stream);
cudaError_t launch_barrier(const RankCtx& c, unsigned* epoch_word, cudaStream_t stream);

// One-time per process: raise the dynamic shared memory limit of every kernel.
cudaError_t configure_kernels(int max_smem);

}  // namespace afdep
