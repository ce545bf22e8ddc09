// tensor::backend::cuda::ops::* (include/tensor/backend/cuda/ops.hpp:12-154) with the reference's exact
// signatures, each forwarding to the C-ABI entry point that replaces it.  The context comes from the current
// device (shim_ctx.hpp); errors surface as CudaError.
//
// Differences a caller can observe, all stated here:
//   * rms_norm_bwd does not produce `dw` (left untouched): every caller in the reference discards it
//     (src/base/arch/qwen2.cu:207,240,298).
//   * sdpa_fwd / sdpa_bwd never materialise the FP32 [B,Hq,T,T] probabilities.  The caller's `attn_w` buffer,
//     which the reference only ever passes from one to the other (qwen2.cu:114-121,266-276), carries instead the
//     per-row log-sum-exp [B,Hq,T] and a BF16 copy of the forward output; that needs T >= 1 + head_dim / 2.
//   * embed_bwd is not on the LoRA path (the embedding is frozen, nothing calls it) and is refused.
#include <tensor/backend/cuda/ops.hpp>

#include <stdexcept>

#include "shim_ctx.hpp"

namespace tensor::backend::cuda::ops {

using ta_shim::as_stream;
using ta_shim::check;
using ta_shim::ctx;

void rms_norm_fwd(const __nv_bfloat16* x, const __nv_bfloat16* w, __nv_bfloat16* out, float* rms_out, int B, int T, int D,
                  float eps, cudaStream_t stream) {
    check(ta_rms_norm_fwd(ctx(), x, w, out, rms_out, B * T, D, eps, as_stream(stream)), "rms_norm_fwd");
}

void rms_norm_bwd(const __nv_bfloat16* dy, const __nv_bfloat16* x, const __nv_bfloat16* w, const float* rms_saved,
                  __nv_bfloat16* dx, float* /*dw: not produced*/, int B, int T, int D, float /*eps*/, cudaStream_t stream) {
    check(ta_rms_norm_bwd(ctx(), dy, x, w, rms_saved, dx, nullptr, B * T, D, as_stream(stream)), "rms_norm_bwd");
}

void rope_fwd(__nv_bfloat16* x, int B, int T, int H, int head_dim, float theta, cudaStream_t stream) {
    check(ta_rope(ctx(), x, H, nullptr, 0, B, T, head_dim, theta, 0, as_stream(stream)), "rope_fwd");
}

void rope_bwd(__nv_bfloat16* dx, int B, int T, int H, int head_dim, float theta, cudaStream_t stream) {
    check(ta_rope(ctx(), dx, H, nullptr, 0, B, T, head_dim, theta, 1, as_stream(stream)), "rope_bwd");
}

namespace {
// Layout of the borrowed attn_w buffer: lse [B*Hq*T] floats, padded to 16 bytes, then out [B*T][Hq*hd] BF16.
struct AttnCache {
    float* lse;
    __nv_bfloat16* out;
};
AttnCache attn_cache(float* attn_w, int B, int T, int Hq, int hd) {
    if (T < 1 + hd / 2)
        throw std::runtime_error("sdpa: the attn_w buffer is too small to carry lse + output for T < 1 + head_dim/2");
    const std::size_t n = (std::size_t(B) * Hq * T + 3) / 4 * 4;
    return AttnCache{attn_w, reinterpret_cast<__nv_bfloat16*>(attn_w + n)};
}
}  // namespace

void sdpa_fwd(const __nv_bfloat16* Q, const __nv_bfloat16* K, const __nv_bfloat16* V, __nv_bfloat16* out, float* attn_w, int B,
              int T, int Hq, int Hkv, int head_dim, const Device& dev) {
    const AttnCache c = attn_cache(attn_w, B, T, Hq, head_dim);
    check(ta_flash_attn_fwd(ctx(), Q, K, V, out, c.lse, B, T, Hq, Hkv, head_dim, as_stream(dev.stream())), "sdpa_fwd");
    CUDA_CHECK(cudaMemcpyAsync(c.out, out, std::size_t(B) * T * Hq * head_dim * sizeof(__nv_bfloat16), cudaMemcpyDeviceToDevice,
                               dev.stream()));
}

void sdpa_bwd(const __nv_bfloat16* dout, const __nv_bfloat16* Q, const __nv_bfloat16* K, const __nv_bfloat16* V,
              const float* attn_w, __nv_bfloat16* dQ, __nv_bfloat16* dK, __nv_bfloat16* dV, int B, int T, int Hq, int Hkv,
              int head_dim, const Device& dev) {
    const AttnCache c = attn_cache(const_cast<float*>(attn_w), B, T, Hq, head_dim);
    check(ta_flash_attn_bwd(ctx(), dout, Q, K, V, c.out, c.lse, dQ, dK, dV, nullptr, B, T, Hq, Hkv, head_dim,
                            as_stream(dev.stream())),
          "sdpa_bwd");
}

void silu_mul_fwd(const __nv_bfloat16* gate, const __nv_bfloat16* up, __nv_bfloat16* out, int N, cudaStream_t stream) {
    check(ta_silu_mul_fwd(ctx(), gate, up, out, N, as_stream(stream)), "silu_mul_fwd");
}

void silu_mul_bwd(const __nv_bfloat16* dout, const __nv_bfloat16* gate, const __nv_bfloat16* up, __nv_bfloat16* dgate,
                  __nv_bfloat16* dup, int N, cudaStream_t stream) {
    check(ta_silu_mul_bwd(ctx(), dout, gate, up, dgate, dup, N, as_stream(stream)), "silu_mul_bwd");
}

void cross_entropy_fwd(const __nv_bfloat16* logits, const int* targets, float* loss_out, __nv_bfloat16* dlogits, int N, int V,
                       cudaStream_t stream) {
    // the reference scales the gradient by 1 / rows (src/backend/cuda/ops.cu:1005)
    check(ta_cross_entropy_fwd(ctx(), logits, targets, loss_out, dlogits, N, V, 1.f / float(N), as_stream(stream)),
          "cross_entropy_fwd");
}

void embed_fwd(const __nv_bfloat16* table, const int* tokens, __nv_bfloat16* out, int BT, int D, cudaStream_t stream) {
    check(ta_embed_fwd(ctx(), table, tokens, out, BT, D, as_stream(stream)), "embed_fwd");
}

void embed_bwd(const __nv_bfloat16*, const int*, float*, int, int, cudaStream_t) {
    throw std::runtime_error("embed_bwd: not built - the embedding table is frozen on the LoRA training path");
}

void add_bias(__nv_bfloat16* out, const __nv_bfloat16* bias, int BT, int D, cudaStream_t stream) {
    check(ta_add_bias(ctx(), out, bias, BT, D, as_stream(stream)), "add_bias");
}

void add_inplace(__nv_bfloat16* out, const __nv_bfloat16* delta, int N, cudaStream_t stream) {
    check(ta_add_inplace(ctx(), out, delta, N, as_stream(stream)), "add_inplace");
}

void lora_add(__nv_bfloat16* out, const __nv_bfloat16* lora_delta, float scale, int N, cudaStream_t stream) {
    check(ta_lora_add(ctx(), out, lora_delta, scale, N, as_stream(stream)), "lora_add");
}

void cast_bf16_to_f32(const __nv_bfloat16* src, float* dst, int N, cudaStream_t s) {
    check(ta_cast_bf16_to_f32(ctx(), src, dst, N, as_stream(s)), "cast_bf16_to_f32");
}

void cast_f32_to_bf16(const float* src, __nv_bfloat16* dst, int N, cudaStream_t s) {
    check(ta_cast_f32_to_bf16(ctx(), src, dst, N, as_stream(s)), "cast_f32_to_bf16");
}

void adamw_step(float* master, __nv_bfloat16* working, float* m, float* v, const float* grad, int N, float lr, float beta1,
                float beta2, float eps, float weight_decay, int step, cudaStream_t stream) {
    check(ta_adamw_step(ctx(), master, working, m, v, grad, N, lr, beta1, beta2, eps, weight_decay, step, as_stream(stream)),
          "adamw_step");
}

void sum_sq_into(const float* g, float* accum, int N, cudaStream_t s) {
    check(ta_sum_sq_into(ctx(), g, accum, N, as_stream(s)), "sum_sq_into");
}

}  // namespace tensor::backend::cuda::ops
