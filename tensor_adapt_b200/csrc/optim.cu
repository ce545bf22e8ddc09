// Optimiser side of the step: sum of squares (gradient norm), clip scale and AdamW over FLAT
// parameter arenas.  All LoRA tensors of a model live back to back in five parallel arrays
// (FP32 master / m / v / grad and the BF16 working copy), so the 24*L launches of the reference
// (8L single-block norm kernels, 8L scale kernels, 8L AdamW kernels) collapse into three.
// Reductions are two-stage with a fixed order: repeated runs give identical bits.
#include <algorithm>
#include <cmath>

#include "ctx.h"
#include "ptx.cuh"

namespace ta {
namespace {

constexpr int kRedThreads = 256;
constexpr int kMaxRedBlocks = 1024;

__global__ void __launch_bounds__(kRedThreads) sum_sq_partial_kernel(const float* __restrict__ g, long n,
                                                                     float* __restrict__ partial) {
    __shared__ float red[kRedThreads / 32];
    // contiguous chunk per block so the summation order is a function of (n, gridDim) only
    const long per = (n + gridDim.x - 1) / gridDim.x;
    const long lo = per * blockIdx.x, hi = min(n, lo + per);
    float s = 0.f;
    for (long i = lo + threadIdx.x; i < hi; i += kRedThreads) {
        const float v = g[i];
        s += v * v;
    }
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < kRedThreads / 32; w++) t += red[w];
        partial[blockIdx.x] = t;
    }
}

// stats[0] = norm, stats[1] = clip scale (1 when norm <= max_norm or max_norm <= 0);
// accum (optional) += sum of squares, the contract of ops::sum_sq_into.
__global__ void sum_sq_final_kernel(const float* __restrict__ partial, int nblocks, float max_norm,
                                    float* __restrict__ stats, float* __restrict__ accum) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    float t = 0.f;
    for (int i = 0; i < nblocks; i++) t += partial[i];
    if (accum) *accum += t;
    if (stats) {
        const float norm = sqrtf(t);
        stats[0] = norm;
        stats[1] = (max_norm > 0.f && norm > max_norm) ? max_norm / (norm + 1e-6f) : 1.f;
    }
}

__global__ void adamw_kernel(float* __restrict__ master, __nv_bfloat16* __restrict__ working, float* __restrict__ m,
                             float* __restrict__ v, const float* __restrict__ grad, long n, float lr, float b1,
                             float b2, float eps, float wd, float bc1, float bc2,
                             const float* __restrict__ stats) {
    const float gs = stats ? stats[1] : 1.f;
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < n; i += long(gridDim.x) * blockDim.x) {
        const float g = grad[i] * gs;
        const float mi = b1 * m[i] + (1.f - b1) * g;
        const float vi = b2 * v[i] + (1.f - b2) * g * g;
        m[i] = mi;
        v[i] = vi;
        const float mhat = mi / bc1, vhat = vi / bc2;
        const float w = master[i];
        const float p = w - lr * (mhat / (sqrtf(vhat) + eps) + wd * w);
        master[i] = p;
        working[i] = __float2bfloat16(p);
    }
}

__global__ void scale_kernel(float* __restrict__ g, long n, const float* __restrict__ stats) {
    const float s = stats[1];
    if (s == 1.f) return;
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < n; i += long(gridDim.x) * blockDim.x) g[i] *= s;
}

int sum_sq(ta_ctx* ctx, const float* g, long n, float max_norm, float* stats, float* accum, cudaStream_t s) {
    const int blocks = int(std::max<long>(1, std::min<long>(kMaxRedBlocks, (n + 4095) / 4096)));
    void* ws = nullptr;
    if (int rc = get_workspace(ctx, kMaxRedBlocks * sizeof(float), &ws)) return rc;
    sum_sq_partial_kernel<<<blocks, kRedThreads, 0, s>>>(g, n, static_cast<float*>(ws));
    TA_LAUNCH_CHECK(ctx, "sum_sq_partial_kernel");
    sum_sq_final_kernel<<<1, 32, 0, s>>>(static_cast<float*>(ws), blocks, max_norm, stats, accum);
    TA_LAUNCH_CHECK(ctx, "sum_sq_final_kernel");
    return TA_OK;
}

}  // namespace
}  // namespace ta

using namespace ta;

extern "C" {

int ta_sum_sq_into(ta_ctx* ctx, const float* g, float* accum, long n, void* stream) {
    if (!ctx || !g || !accum || n < 0) return fail(ctx, TA_ERR_INVALID, "sum_sq_into: null argument");
    if (n == 0) return TA_OK;
    return sum_sq(ctx, g, n, 0.f, nullptr, accum, static_cast<cudaStream_t>(stream));
}

int ta_adamw_step(ta_ctx* ctx, float* master, void* working, float* m, float* v, const float* grad, long n, float lr,
                  float beta1, float beta2, float eps, float weight_decay, int step, void* stream) {
    if (!ctx || !master || !working || !m || !v || !grad || n < 0 || step < 1)
        return fail(ctx, TA_ERR_INVALID, "adamw_step: null argument or step < 1");
    if (n == 0) return TA_OK;
    const float bc1 = 1.f - std::pow(beta1, float(step)), bc2 = 1.f - std::pow(beta2, float(step));
    const unsigned grid = unsigned(std::min<long>((n + 255) / 256, long(ctx->sm_count) * 8));
    adamw_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        master, static_cast<__nv_bfloat16*>(working), m, v, grad, n, lr, beta1, beta2, eps, weight_decay, bc1, bc2,
        nullptr);
    TA_LAUNCH_CHECK(ctx, "adamw_kernel");
    return TA_OK;
}

int ta_gradnorm_clip_adamw(ta_ctx* ctx, float* master, void* working, float* m, float* v, float* grad, long n, float lr,
                           float beta1, float beta2, float eps, float weight_decay, int step, float max_norm,
                           float* stats_dev, int scale_grads_in_place, void* stream) {
    if (!ctx || !master || !working || !m || !v || !grad || !stats_dev || n <= 0 || step < 1)
        return fail(ctx, TA_ERR_INVALID, "gradnorm_clip_adamw: null argument, n <= 0 or step < 1");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (int rc = sum_sq(ctx, grad, n, max_norm, stats_dev, nullptr, s)) return rc;
    const unsigned grid = unsigned(std::min<long>((n + 255) / 256, long(ctx->sm_count) * 8));
    const float bc1 = 1.f - std::pow(beta1, float(step)), bc2 = 1.f - std::pow(beta2, float(step));
    if (scale_grads_in_place) {
        // what clip_gradients leaves behind: the gradient buffers themselves are scaled
        scale_kernel<<<grid, 256, 0, s>>>(grad, n, stats_dev);
        TA_LAUNCH_CHECK(ctx, "scale_kernel");
        adamw_kernel<<<grid, 256, 0, s>>>(master, static_cast<__nv_bfloat16*>(working), m, v, grad, n, lr, beta1, beta2,
                                          eps, weight_decay, bc1, bc2, nullptr);
    } else {
        adamw_kernel<<<grid, 256, 0, s>>>(master, static_cast<__nv_bfloat16*>(working), m, v, grad, n, lr, beta1, beta2,
                                          eps, weight_decay, bc1, bc2, stats_dev);
    }
    TA_LAUNCH_CHECK(ctx, "adamw_kernel");
    return TA_OK;
}

}  // extern "C"
