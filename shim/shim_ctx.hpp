// Shared plumbing of the drop-in shims: the reference's C++ API carries only a cudaStream_t (ops::*) or a
// Device (everything else), never a library context, so the shims keep ONE ta_ctx per CUDA device of the
// process, created on first use for the device that is current at that moment.
//
// Errors follow the reference's convention (include/tensor/backend/cuda/device.hpp:15-42): a failed call
// throws tensor::backend::cuda::CudaError carrying the library's message.
#pragma once

#include <tensor/backend/cuda/device.hpp>

#include <cuda_runtime.h>

#include <string>

#include "tensor_adapt_b200.h"

namespace ta_shim {

// Context of the current CUDA device (single host thread, like the reference's Device).
ta_ctx* ctx();

// Turns a TA_ERR_* status into the exception the reference's callers already catch.
inline void check(int rc, const char* what) {
    if (rc == TA_OK) return;
    throw tensor::backend::cuda::CudaError(std::string(what) + ": " + ta_last_error(ctx()) + " (status " + std::to_string(rc) + ")");
}

inline void* as_stream(cudaStream_t s) { return static_cast<void*>(s); }

}  // namespace ta_shim
