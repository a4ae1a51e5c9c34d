// Stream-ordered 32-bit memory operations issued by the driver's front end rather than by a
// kernel: a batch of writes that runs after everything queued before it on the stream.  Used to
// signal peers after copy-engine transfers, so an all-gather can run without occupying an SM.
//
// Only the write half is offered.  A stream-ordered *wait* has no time limit: a peer that never
// writes would stall the stream for good, so every wait in this library stays inside a kernel
// with a clock budget (see status.cuh).  The reference batches both writes and waits for its
// in-session all-gather (csrc/kernels/backend/cuda_driver.cu:12-52).
#pragma once
#include <cstdint>
#include <vector>

#include "driver.hpp"

namespace afdep {

struct StreamWrite32 {
    void* address;      // 4-byte aligned device address, local or a mapped peer's
    uint32_t value;
};

// Queue `writes` on `stream` as one batched memory operation.  Each write is preceded by the
// default memory barrier, so data copied earlier on the stream is visible before the value is.
inline void stream_write32_batch(cudaStream_t stream, const std::vector<StreamWrite32>& writes) {
    if (writes.empty()) return;
    std::vector<CUstreamBatchMemOpParams> ops(writes.size());
    for (size_t i = 0; i < writes.size(); ++i) {
        ops[i] = CUstreamBatchMemOpParams{};
        ops[i].writeValue.operation = CU_STREAM_MEM_OP_WRITE_VALUE_32;
        ops[i].writeValue.address = reinterpret_cast<CUdeviceptr>(writes[i].address);
        ops[i].writeValue.value = writes[i].value;
        ops[i].writeValue.flags = CU_STREAM_WRITE_VALUE_DEFAULT;
    }
    static const auto batch = AFDEP_DRV(cuStreamBatchMemOp);
    drv_check(batch(reinterpret_cast<CUstream>(stream), (unsigned)ops.size(), ops.data(), 0), "cuStreamBatchMemOp");
}

}  // namespace afdep
