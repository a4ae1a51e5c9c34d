#include "heap.hpp"

#include <unistd.h>

#include <cstdint>
#include <cstring>

#include "driver.hpp"

namespace afdep {

namespace {

CUmemAllocationProp vmm_prop(int device) {
    CUmemAllocationProp prop;
    std::memset(&prop, 0, sizeof(prop));
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    return prop;
}

void* map_handle(CUmemGenericAllocationHandle h, size_t size, size_t gran, int device) {
    CUdeviceptr ptr = 0;
    drv_check(AFDEP_DRV(cuMemAddressReserve)(&ptr, size, gran, 0, 0), "cuMemAddressReserve");
    CUresult r = AFDEP_DRV(cuMemMap)(ptr, size, 0, h, 0);
    if (r != CUDA_SUCCESS) {
        AFDEP_DRV(cuMemAddressFree)(ptr, size);
        drv_check(r, "cuMemMap");
    }
    CUmemAccessDesc acc;
    std::memset(&acc, 0, sizeof(acc));
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = device;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    r = AFDEP_DRV(cuMemSetAccess)(ptr, size, &acc, 1);
    if (r != CUDA_SUCCESS) {
        AFDEP_DRV(cuMemUnmap)(ptr, size);
        AFDEP_DRV(cuMemAddressFree)(ptr, size);
        drv_check(r, "cuMemSetAccess");
    }
    return reinterpret_cast<void*>(ptr);
}

size_t vmm_granularity(int device) {
    CUmemAllocationProp prop = vmm_prop(device);
    size_t gran = 0;
    drv_check(AFDEP_DRV(cuMemGetAllocationGranularity)(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED),
              "cuMemGetAllocationGranularity");
    return gran;
}

}  // namespace

bool SymmetricHeap::vmm_supported(int device) {
    try {
        int v = 0;
        CUdevice dev;
        drv_check(AFDEP_DRV(cuDeviceGet)(&dev, device), "cuDeviceGet");
        drv_check(AFDEP_DRV(cuDeviceGetAttribute)(&v, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, dev),
                  "cuDeviceGetAttribute");
        if (!v) return false;
        drv_check(AFDEP_DRV(cuDeviceGetAttribute)(&v, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev),
                  "cuDeviceGetAttribute");
        return v != 0;
    } catch (...) {
        return false;
    }
}

SymmetricHeap::SymmetricHeap(int device, size_t bytes, Mode mode) : device_(device), bytes_(bytes), mapped_(bytes), mode_(mode) {
    rt_check(cudaSetDevice(device), "cudaSetDevice");
    rt_check(cudaFree(nullptr), "CUDA context creation");
    if (mode_ == Mode::kVmmFd) {
        const size_t gran = vmm_granularity(device);
        mapped_ = (bytes + gran - 1) / gran * gran;
        CUmemAllocationProp prop = vmm_prop(device);
        CUmemGenericAllocationHandle h = 0;
        drv_check(AFDEP_DRV(cuMemCreate)(&h, mapped_, &prop, 0), "cuMemCreate");
        handle_ = h;
        try {
            local_ = map_handle(h, mapped_, gran, device);
        } catch (...) {
            AFDEP_DRV(cuMemRelease)(h);
            handle_ = 0;
            throw;
        }
    } else {
        rt_check(cudaMalloc(&local_, bytes), "cudaMalloc(symmetric heap)");
    }
}

SymmetricHeap::~SymmetricHeap() {
    try {
        release();
    } catch (...) {
    }
}

int SymmetricHeap::export_fd() {
    if (mode_ != Mode::kVmmFd) throw std::runtime_error("heap was not created with file-descriptor export");
    int fd = -1;
    drv_check(AFDEP_DRV(cuMemExportToShareableHandle)(&fd, handle_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
              "cuMemExportToShareableHandle");
    return fd;
}

std::string SymmetricHeap::export_ipc() {
    if (mode_ != Mode::kCudaIpc) throw std::runtime_error("heap was not created for cudaIpc export");
    cudaIpcMemHandle_t h;
    rt_check(cudaIpcGetMemHandle(&h, local_), "cudaIpcGetMemHandle");
    return std::string(reinterpret_cast<const char*>(&h), sizeof(h));
}

void* SymmetricHeap::import_fd(int fd, size_t mapped_bytes) {
    rt_check(cudaSetDevice(device_), "cudaSetDevice");
    CUmemGenericAllocationHandle h = 0;
    drv_check(AFDEP_DRV(cuMemImportFromShareableHandle)(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
              "cuMemImportFromShareableHandle");
    void* p = nullptr;
    try {
        p = map_handle(h, mapped_bytes, vmm_granularity(device_), device_);
    } catch (...) {
        AFDEP_DRV(cuMemRelease)(h);
        throw;
    }
    imports_.push_back({p, mapped_bytes, h});
    return p;
}

void* SymmetricHeap::import_ipc(const std::string& handle) {
    rt_check(cudaSetDevice(device_), "cudaSetDevice");
    if (handle.size() != sizeof(cudaIpcMemHandle_t)) throw std::runtime_error("malformed cudaIpc handle");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle.data(), sizeof(h));
    void* p = nullptr;
    rt_check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    imports_.push_back({p, 0, 0});
    return p;
}

void SymmetricHeap::release() {
    if (released_) return;
    released_ = true;
    cudaSetDevice(device_);
    for (auto& im : imports_) {
        if (im.handle) {
            AFDEP_DRV(cuMemUnmap)(reinterpret_cast<CUdeviceptr>(im.ptr), im.bytes);
            AFDEP_DRV(cuMemAddressFree)(reinterpret_cast<CUdeviceptr>(im.ptr), im.bytes);
            AFDEP_DRV(cuMemRelease)(im.handle);
        } else {
            cudaIpcCloseMemHandle(im.ptr);
        }
    }
    imports_.clear();
    if (local_) {
        if (mode_ == Mode::kVmmFd) {
            AFDEP_DRV(cuMemUnmap)(reinterpret_cast<CUdeviceptr>(local_), mapped_);
            AFDEP_DRV(cuMemAddressFree)(reinterpret_cast<CUdeviceptr>(local_), mapped_);
            AFDEP_DRV(cuMemRelease)(handle_);
        } else {
            cudaFree(local_);
        }
        local_ = nullptr;
    }
}

}  // namespace afdep
