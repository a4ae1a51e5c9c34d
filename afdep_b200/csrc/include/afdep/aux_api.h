// Secondary primitives on the symmetric heap's auxiliary region: neighbour send/recv with
// credits, all-gather, and remote row fetch.  NVLink only; every wait is bounded.
//
// Auxiliary region of a rank (offset Geometry::aux_off, Geometry::aux_bytes long):
//   [0, 4096)        signal words, uint32:
//                      [0, 8)    gather flags, one per source rank
//                      [8, 16)   send flags:  send_flag[src] = sequence number of the last message from src
//                      [16, 24)  ack words:   ack[dst] = sequence number of the last message dst consumed
//   [4096, ...)      data, used by one primitive at a time:
//                      all-gather   two sets (gather parity) of one slot per rank
//                      send/recv    per source rank a ring of `inflight` message slots
//                      row fetch    this rank's shard of the table
//
// Counterparts in the reference: pp_send_impl / pp_recv_impl (impls/pp_send_recv.cuh), the
// host-driven AGRS all_gather (csrc/elastic/buffer.hpp:325-474) and engram_fetch_impl
// (impls/engram_fetch.cuh), all of which need NCCL GIN or driver batch copies there.
#pragma once
#include <cuda_runtime.h>

#include "kernels.h"

namespace afdep {

constexpr int kAuxSignalBytes = 4096;

struct AuxSeq {            // device-resident sequence numbers (never reset)
    unsigned* gather;      // exchanges of all_gather completed
    unsigned* sent;        // [kMaxRanks] messages sent to each peer
    unsigned* received;    // [kMaxRanks] messages consumed from each peer
    unsigned* ticket;      // [3] CTA completion counters: gather push, send, receive (a send may overlap a receive;
                           // two sends, or two receives, of one Buffer must not overlap each other)
};

// Copy `bytes` from `src` into slot [rank] of every peer's data area and raise the gather flag.
cudaError_t launch_allgather_push(const RankCtx& c, const AuxSeq& seq, const void* src, size_t bytes, size_t slot_bytes,
                                  int ctas, cudaStream_t stream);
// Wait until every rank's slot of this rank's data area carries the current gather.
cudaError_t launch_allgather_wait(const RankCtx& c, const AuxSeq& seq, cudaStream_t stream);

// After the wait: copies the world x `bytes` contributions of the gather just completed out of the heap.
cudaError_t launch_allgather_copy_out(const RankCtx& c, const AuxSeq& seq, void* out, size_t bytes, size_t slot_bytes, cudaStream_t stream);

// Neighbour message: waits for credit (the peer consumed message seq - inflight), copies, flags.
cudaError_t launch_p2p_send(const RankCtx& c, const AuxSeq& seq, int dst, const void* src, size_t bytes, size_t slot_bytes,
                            int inflight, int ctas, cudaStream_t stream);
// Waits for the next message from `src_rank`, copies it out and returns the credit.
cudaError_t launch_p2p_recv(const RankCtx& c, const AuxSeq& seq, int src_rank, void* dst, size_t bytes, size_t slot_bytes,
                            int inflight, int ctas, cudaStream_t stream);
// Once per device: raise the dynamic shared memory limit of the copy pipelines.
cudaError_t configure_aux();

// out[i] = row `idx[i] % rows_per_rank` of the table shard in rank `idx[i] / rows_per_rank`'s data area.
cudaError_t launch_fetch_rows(const RankCtx& c, const long long* idx, int n, int rows_per_rank, int row_bytes, void* out,
                              int ctas, cudaStream_t stream);

}  // namespace afdep
