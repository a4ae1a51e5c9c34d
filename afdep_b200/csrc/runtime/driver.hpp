// CUDA driver entry points resolved at run time through the runtime library
// (cudaGetDriverEntryPoint), so the extension links against nothing but cudart and still
// imports on a machine without a driver.  The reference dlopen()s libcuda for the same
// reason (csrc/utils/lazy_driver.hpp).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

namespace afdep {

inline void* driver_symbol(const char* name) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || fn == nullptr) {
        cudaGetLastError();
        throw std::runtime_error(std::string("CUDA driver entry point unavailable: ") + name);
    }
    return fn;
}

#define AFDEP_DRV(name) (reinterpret_cast<decltype(&name)>(::afdep::driver_symbol(#name)))

inline void drv_check(CUresult r, const char* what) {
    if (r != CUDA_SUCCESS) {
        const char* msg = nullptr;
        try {
            AFDEP_DRV(cuGetErrorString)(r, &msg);
        } catch (...) {
        }
        throw std::runtime_error(std::string(what) + " failed: " + (msg ? msg : "unknown driver error") + " (" +
                                 std::to_string((int)r) + ")");
    }
}

inline void rt_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) {
        cudaGetLastError();
        throw std::runtime_error(std::string(what) + " failed: " + cudaGetErrorString(e));
    }
}

}  // namespace afdep
