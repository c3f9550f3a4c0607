// Host-side CUDA helpers: error mapping, lazy "is there a usable device" probe, and driver
// API entry points fetched through the runtime so the library loads on machines without a
// driver (the static runtime resolves libcuda only when first used).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "../core/log.h"
#include "xccl/xccl.h"

namespace xccl {

// true when at least one CUDA device can be used by this process (cached)
bool cuda_available();

// Fetches a driver entry point by name ("cuMemCreate"); nullptr when there is no driver.
void *cuda_driver_fn(const char *name);

inline xccl_status_t cuda_status(cudaError_t e)
{
    switch (e) {
    case cudaSuccess: return XCCL_OK;
    case cudaErrorNotReady: return XCCL_INPROGRESS;
    case cudaErrorMemoryAllocation: return XCCL_ERR_NO_MEMORY;
    case cudaErrorInvalidValue: return XCCL_ERR_INVALID_PARAM;
    default: return XCCL_ERR_NO_MESSAGE;
    }
}

}  // namespace xccl

#define XCCL_CUDA_CHECK(expr)                                                                    \
    do {                                                                                         \
        cudaError_t _e = (expr);                                                                 \
        if (_e != cudaSuccess) {                                                                 \
            xccl_error("%s failed: %s", #expr, cudaGetErrorString(_e));                          \
            return ::xccl::cuda_status(_e);                                                      \
        }                                                                                        \
    } while (0)

#define XCCL_CU_CHECK(expr)                                                                      \
    do {                                                                                         \
        CUresult _r = (expr);                                                                    \
        if (_r != CUDA_SUCCESS) {                                                                \
            xccl_error("%s failed: CUresult %d", #expr, (int)_r);                                \
            return XCCL_ERR_NO_MESSAGE;                                                          \
        }                                                                                        \
    } while (0)

// Declares a local function pointer `name` of the driver API type and fails when missing.
#define XCCL_DRIVER_FN(name)                                                                     \
    auto name = reinterpret_cast<decltype(&::name)>(::xccl::cuda_driver_fn(#name));              \
    if (name == nullptr) {                                                                       \
        xccl_error("CUDA driver entry point %s is not available", #name);                        \
        return XCCL_ERR_UNSUPPORTED;                                                             \
    }
