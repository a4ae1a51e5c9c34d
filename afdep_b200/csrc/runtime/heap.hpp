// Symmetric heap: one physical allocation per rank that every peer of the NVLink domain maps
// into its own address space, so kernels can store to and load from any rank with ordinary
// pointers.  Preferred backing is the CUDA virtual-memory API with POSIX file-descriptor
// export (the descriptors travel between processes over a Unix socket, done in Python);
// cudaIpc handles on a cudaMalloc block are the fallback, and a plain cudaMalloc serves the
// single-process loopback world.  Replaces the reference's NCCL window registration
// (csrc/kernels/backend/nccl.cu:64-168); its own VMM helper (csrc/utils/shared_memory.hpp)
// ships unused.
#pragma once
#include <cstddef>
#include <string>
#include <vector>

namespace afdep {

class SymmetricHeap {
public:
    enum class Mode { kVmmFd, kCudaIpc, kPlain };

    SymmetricHeap(int device, size_t bytes, Mode mode);
    ~SymmetricHeap();
    SymmetricHeap(const SymmetricHeap&) = delete;
    SymmetricHeap& operator=(const SymmetricHeap&) = delete;

    void* local() const { return local_; }
    size_t bytes() const { return bytes_; }          // requested size
    size_t mapped_bytes() const { return mapped_; }  // after granularity rounding
    Mode mode() const { return mode_; }

    int export_fd();                 // kVmmFd: a new descriptor, owned by the caller
    std::string export_ipc();        // kCudaIpc: the 64-byte handle
    void* import_fd(int fd, size_t mapped_bytes);
    void* import_ipc(const std::string& handle);
    void release();                  // unmap peers, free the local block; idempotent

    static bool vmm_supported(int device);

private:
    struct Import {
        void* ptr;
        size_t bytes;
        unsigned long long handle;   // CUmemGenericAllocationHandle, 0 for cudaIpc
    };
    int device_;
    size_t bytes_, mapped_;
    Mode mode_;
    void* local_ = nullptr;
    unsigned long long handle_ = 0;
    std::vector<Import> imports_;
    bool released_ = false;
};

}  // namespace afdep
