// tensor::backend::cuda::Device over the CUDA runtime (include/tensor/backend/cuda/device.hpp:52-79,
// src/backend/cuda/device.cu:25-48), plus the per-device library context the other shims share.
// No cuBLAS handle is created: nothing behind these shims calls cuBLAS, so cublas() returns nullptr.
#include "shim_ctx.hpp"

#include <map>
#include <utility>

namespace ta_shim {

ta_ctx* ctx() {
    static std::map<int, ta_ctx*> per_device;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) throw tensor::backend::cuda::CudaError("cudaGetDevice failed");
    auto it = per_device.find(dev);
    if (it != per_device.end()) return it->second;
    ta_ctx* c = nullptr;
    const int rc = ta_ctx_create(dev, &c);
    if (rc != TA_OK)
        throw tensor::backend::cuda::CudaError(rc == TA_ERR_UNSUPPORTED
                                                   ? "this build runs on sm_100 (B200) devices only; there is no fallback path"
                                                   : "ta_ctx_create failed (status " + std::to_string(rc) + ")");
    per_device[dev] = c;
    return c;
}

}  // namespace ta_shim

namespace tensor::backend::cuda {

Device Device::open(const std::string& spec) {
    int id = 0;
    if (spec.rfind("cuda:", 0) == 0) id = std::stoi(spec.substr(5));
    else if (spec != "cuda") throw CudaError("unsupported device spec '" + spec + "' (expected cuda or cuda:N)");
    CUDA_CHECK(cudaSetDevice(id));
    Device d;
    d.id_ = id;
    int major = 0;
    CUDA_CHECK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, id));
    d.sm_major_ = major;
    CUDA_CHECK(cudaStreamCreate(&d.stream_));
    ta_shim::ctx();   // fails here, loudly, on anything but sm_100
    return d;
}

void Device::sync() const { CUDA_CHECK(cudaStreamSynchronize(stream_)); }

Device::Device(Device&& o) noexcept
    : id_(o.id_), sm_major_(o.sm_major_), cublas_(o.cublas_), stream_(o.stream_) {
    o.cublas_ = nullptr;
    o.stream_ = nullptr;
}

Device& Device::operator=(Device&& o) noexcept {
    if (this != &o) {
        if (stream_) cudaStreamDestroy(stream_);
        id_ = o.id_; sm_major_ = o.sm_major_; cublas_ = o.cublas_; stream_ = o.stream_;
        o.cublas_ = nullptr; o.stream_ = nullptr;
    }
    return *this;
}

Device::~Device() {
    if (stream_) cudaStreamDestroy(stream_);
}

}  // namespace tensor::backend::cuda
