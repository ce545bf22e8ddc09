// tensor::backend::cuda::Tensor (include/tensor/backend/cuda/tensor.hpp:25-77, src/backend/cuda/tensor.cu:20-128)
// as a plain owner of one cudaMalloc block, and gemm_bf16 (tensor.hpp:85-91, tensor.cu:144-166) on the
// library's tcgen05 GEMM for the two operand arrangements the training path uses.
#include <tensor/backend/cuda/tensor.hpp>

#include <stdexcept>
#include <utility>

#include "shim_ctx.hpp"

namespace tensor::backend::cuda {

Tensor Tensor::empty(const Shape& shape, DType dtype, const Device& dev) {
    Tensor t;
    t.shape_ = shape; t.dtype_ = dtype; t.device_id_ = dev.id();
    const std::size_t n = t.nbytes();
    if (n) CUDA_CHECK(cudaMalloc(&t.ptr_, n));
    return t;
}

Tensor Tensor::zeros(const Shape& shape, DType dtype, const Device& dev) {
    Tensor t = empty(shape, dtype, dev);
    if (t.ptr_) CUDA_CHECK(cudaMemsetAsync(t.ptr_, 0, t.nbytes(), dev.stream()));
    return t;
}

Tensor Tensor::from_host(const TensorView& src, const Device& dev) {
    Tensor t = empty(src.shape, src.dtype, dev);
    if (t.ptr_) {
        CUDA_CHECK(cudaMemcpyAsync(t.ptr_, src.data, t.nbytes(), cudaMemcpyHostToDevice, dev.stream()));
        CUDA_CHECK(cudaStreamSynchronize(dev.stream()));   // the source may be a temporary, as in the reference's callers
    }
    return t;
}

Tensor Tensor::empty_bf16(const Shape& shape, const Device& dev) { return empty(shape, DType::BF16, dev); }
Tensor Tensor::empty_f32(const Shape& shape, const Device& dev) { return empty(shape, DType::F32, dev); }
Tensor Tensor::zeros_f32(const Shape& shape, const Device& dev) { return zeros(shape, DType::F32, dev); }

template <typename T>
static std::vector<T> to_host(const Tensor& t, DType want, const char* name) {
    if (t.dtype() != want) throw std::runtime_error(std::string(name) + ": dtype mismatch");
    std::vector<T> h(t.numel());
    if (!h.empty()) CUDA_CHECK(cudaMemcpy(h.data(), t.data(), t.nbytes(), cudaMemcpyDeviceToHost));
    return h;
}

std::vector<__nv_bfloat16> Tensor::to_host_bf16() const { return to_host<__nv_bfloat16>(*this, DType::BF16, "to_host_bf16"); }
std::vector<float> Tensor::to_host_f32() const { return to_host<float>(*this, DType::F32, "to_host_f32"); }
std::vector<uint32_t> Tensor::to_host_u32() const { return to_host<uint32_t>(*this, DType::I32, "to_host_u32"); }

void Tensor::zero_(const Device& dev) {
    if (ptr_) CUDA_CHECK(cudaMemsetAsync(ptr_, 0, nbytes(), dev.stream()));
}

Tensor::Tensor(Tensor&& o) noexcept
    : ptr_(o.ptr_), shape_(std::move(o.shape_)), dtype_(o.dtype_), device_id_(o.device_id_) {
    o.ptr_ = nullptr;
}

Tensor& Tensor::operator=(Tensor&& o) noexcept {
    if (this != &o) {
        if (ptr_) cudaFree(ptr_);
        ptr_ = o.ptr_; shape_ = std::move(o.shape_); dtype_ = o.dtype_; device_id_ = o.device_id_;
        o.ptr_ = nullptr;
    }
    return *this;
}

Tensor::~Tensor() {
    if (ptr_) cudaFree(ptr_);
}

// The reference passes cuBLAS (column-major) arguments.  In row-major terms the two calls of the training
// path are
//   transA, !transB (src/base/arch/qwen2.cu:21-30):  C[N][M] = alpha * B[N][K] . A[M][K]^T          y = x.W^T
//   !transA, !transB (qwen2.cu:32-41):               C[N][M] = alpha * B[N][K] . A[K][M] + beta*C   dx = dy.W
// with beta 0 or 1.  Other arrangements are not on the path and are refused.
void gemm_bf16(const Device& dev, const GemmParams& p, const __nv_bfloat16* A, int lda, const __nv_bfloat16* B, int ldb,
               __nv_bfloat16* C, int ldc) {
    if (p.transB || (p.beta != 0.f && p.beta != 1.f))
        throw std::runtime_error("gemm_bf16: only the proj_fwd / proj_bwd_x operand arrangements (beta 0 or 1) are built");
    const void* residual = p.beta == 1.f ? C : nullptr;
    ta_shim::check(ta_gemm_bf16(ta_shim::ctx(), p.N, p.M, p.K, p.alpha, B, ldb, 0, A, lda, p.transA ? 0 : 1, nullptr, residual, C, ldc,
                                ta_shim::as_stream(dev.stream())),
                   "gemm_bf16");
}

// FP32 GEMMs appear in the reference only inside AdapterModel::apply_lora_bwd, on FP32 copies of BF16 tensors
// (src/adapter/adapter_model.cu:155-207); that whole function is one library call here (see adapter_model.cpp).
void gemm_f32(const Device&, const GemmParams&, const float*, int, const float*, int, float*, int) {
    throw std::runtime_error("gemm_f32: not built - the LoRA gradient products run inside AdapterModel::apply_lora_bwd");
}

}  // namespace tensor::backend::cuda
