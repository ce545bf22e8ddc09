/* tensor_adapt_b200 - C ABI of the B200-native LoRA training hot path.
 *
 * Drop-in boundary for carbon-os/tensor-adapt's CUDA backend and trainer: every entry point
 * below names the reference interface it replaces (file:line inside the reference tree).  The
 * reference has no FFI layer of its own; its boundary is the C++ API in include/tensor/, so each
 * function here is what a thin C++ shim with the reference's name and signature would call
 * (INTEGRATION.md shows those shims).
 *
 * Conventions
 *   - plain pointers and sizes only; `void*` data pointers are DEVICE pointers unless a parameter
 *     is documented as host memory; BF16 tensors are row-major `__nv_bfloat16`.
 *   - `stream` is a `cudaStream_t` passed as `void*` (NULL = the legacy default stream).
 *   - every function returns TA_OK (0) or a negative TA_ERR_* code and never throws; the message is
 *     available from ta_last_error().  Launches are asynchronous unless documented otherwise.
 *   - there is no CPU fallback: without an sm_100 device ta_ctx_create() fails with
 *     TA_ERR_UNSUPPORTED / TA_ERR_CUDA and nothing else can be called.
 */
#ifndef TENSOR_ADAPT_B200_H
#define TENSOR_ADAPT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TA_OK                  0
#define TA_ERR_INVALID        -1   /* bad argument (null, size, alignment)                       */
#define TA_ERR_CUDA           -2   /* a CUDA runtime / driver call failed                        */
#define TA_ERR_UNSUPPORTED    -3   /* not an sm_100 device, or a shape this build does not cover */
#define TA_ERR_DEVICE_TIMEOUT -4   /* a bounded wait inside a kernel ran out (ta_device_status)  */
#define TA_ERR_NOMEM          -5
#define TA_ERR_IO             -6

typedef struct ta_ctx ta_ctx;

/* ── context ───────────────────────────────────────────────────────────────────────────────
 * Replaces backend::cuda::Device (include/tensor/backend/cuda/device.hpp:52-79,
 * src/backend/cuda/device.cu:25-48): selects the device, checks it is sm_100, owns the status
 * word of the bounded device waits, a scratch workspace and the TMA tensor-map cache. */
int ta_ctx_create(int device, ta_ctx** out);
int ta_ctx_destroy(ta_ctx* ctx);
/* Use caller-owned scratch instead of the context's own (which grows with cudaMalloc on demand).
 * Pass NULL to return to the owned workspace. */
int ta_ctx_set_workspace(ta_ctx* ctx, void* workspace, size_t bytes);
const char* ta_last_error(const ta_ctx* ctx);
/* Synchronous read (and reset) of the device status word: TA_OK, or TA_ERR_DEVICE_TIMEOUT with
 * *status = the code of the wait that gave up.  The CUDA context stays usable either way. */
int ta_device_status(ta_ctx* ctx, int* status);
/* Kernels launched through this context so far. */
long ta_launch_count(const ta_ctx* ctx);

/* ── row / element-wise kernels (replace ops::* of include/tensor/backend/cuda/ops.hpp) ────── */

/* ops::rms_norm_fwd (ops.hpp:12-18, src/backend/cuda/ops.cu:59-107). rows = B*T. rms_out may be NULL. */
int ta_rms_norm_fwd(ta_ctx* ctx, const void* x, const void* w, void* out, float* rms_out, int rows, int D, float eps,
                    void* stream);
/* ops::rms_norm_bwd (ops.hpp:20-28, ops.cu:113-170) without the `dw` output, which every caller in the
 * reference discards (src/base/arch/qwen2.cu:207,240,298).  If add_to != NULL the result is
 * dx = bf16(add_to + bf16(dx_norm)): the residual-gradient add (ops::add_inplace) that follows each
 * rms_norm_bwd in Qwen2Base::backward (qwen2.cu:246,304), fused; dx may alias add_to. */
int ta_rms_norm_bwd(ta_ctx* ctx, const void* dy, const void* x, const void* w, const float* rms_saved, void* dx,
                    const void* add_to, int rows, int D, void* stream);
/* ops::rope_fwd / ops::rope_bwd (ops.hpp:31-41, ops.cu:176-204): in-place adjacent-pair rotation of
 * up to two tensors [B*T, H*head_dim] (Q and K) in one launch; inverse != 0 is the backward. */
int ta_rope(ta_ctx* ctx, void* q, int Hq, void* k, int Hk, int B, int T, int head_dim, float theta, int inverse,
            void* stream);
/* ops::silu_mul_fwd / ops::silu_mul_bwd (ops.hpp:73-87, ops.cu:913-952). n = element count. */
int ta_silu_mul_fwd(ta_ctx* ctx, const void* gate, const void* up, void* out, long n, void* stream);
int ta_silu_mul_bwd(ta_ctx* ctx, const void* dout, const void* gate, const void* up, void* dgate, void* dup, long n,
                    void* stream);
/* ops::cross_entropy_fwd (ops.hpp:90-96, ops.cu:958-1020). dlogits may be NULL (loss only) or alias
 * logits.  inv_count is the gradient scale: the reference uses 1/rows (ops.cu:1005); a micro-batched
 * or data-parallel step passes 1/(global token count). Targets < 0 behave as in the reference
 * (loss = logsumexp, gradient still softmax*inv_count). */
int ta_cross_entropy_fwd(ta_ctx* ctx, const void* logits, const int* targets, float* loss_out, void* dlogits, int rows,
                         int V, float inv_count, void* stream);
/* ops::embed_fwd (ops.hpp:99-104, ops.cu:1026-1045). */
int ta_embed_fwd(ta_ctx* ctx, const void* table, const int* tokens, void* out, int BT, int D, void* stream);
/* ops::add_bias (ops.hpp:114-118, ops.cu:1062-1081). */
int ta_add_bias(ta_ctx* ctx, void* out, const void* bias, long rows, int D, void* stream);
/* ops::add_inplace / ops::lora_add (ops.hpp:121-132, ops.cu:1087-1113). */
int ta_add_inplace(ta_ctx* ctx, void* out, const void* delta, long n, void* stream);
int ta_lora_add(ta_ctx* ctx, void* out, const void* delta, float scale, long n, void* stream);
/* ops::cast_bf16_to_f32 / ops::cast_f32_to_bf16 (ops.hpp:135-136, ops.cu:1119-1133). */
int ta_cast_bf16_to_f32(ta_ctx* ctx, const void* src, float* dst, long n, void* stream);
int ta_cast_f32_to_bf16(ta_ctx* ctx, const float* src, void* dst, long n, void* stream);

/* ── GEMM ──────────────────────────────────────────────────────────────────────────────────
 * gemm_bf16 (include/tensor/backend/cuda/tensor.hpp:85-91, src/backend/cuda/tensor.cu:144-166) for
 * the row-major products the training step uses, on tcgen05/TMEM fed by TMA:
 *     C[M,N] = alpha * A.B  (+ bias[N]) (+ residual[M,N])          BF16 in, FP32 accumulate, BF16 out
 * a_layout / b_layout: 0 = "K-major" (A is [M][K], B is [N][K]: the reference's proj_fwd y = x.W^T,
 * qwen2.cu:21-30), 1 = "MN-major" (A is [K][M], B is [K][N]: proj_bwd_x dx = dy.W, qwen2.cu:32-41).
 * lda/ldb/ldc are row pitches in elements (multiples of 8). bias/residual may be NULL. */
int ta_gemm_bf16(ta_ctx* ctx, int M, int N, int K, float alpha, const void* A, long lda, int a_layout, const void* B,
                 long ldb, int b_layout, const void* bias, const void* residual, void* C, long ldc, void* stream);
/* gemm_f32 as used for the LoRA gradients (tensor.hpp:93-99, src/adapter/adapter_model.cu:166-207):
 *     C[M,N] (+)= alpha * sum_k A[k][m] * B[k][n]     BF16 operands (both token-major), FP32 output,
 * contraction over the K = token dimension split across CTAs with a fixed-order reduction.
 * transpose_out != 0 stores C^T (C is then [N][ldc]). */
int ta_gemm_tokens_f32(ta_ctx* ctx, int M, int N, int K, float alpha, const void* A, long lda, const void* B, long ldb,
                       float* C, long ldc, int accumulate, int transpose_out, void* stream);

/* ── LoRA-augmented projection ─────────────────────────────────────────────────────────────
 * proj_fwd + ops::add_bias + AdapterModel::apply_lora_fwd (src/base/arch/qwen2.cu:21-30,95-108;
 * src/adapter/adapter_model.cu:96-129) as one fused product:
 *     y[BT,out] = x.W^T (+ bias) + scale*(x.A^T).B^T (+ residual)
 * x [BT,in], W [out,in], A [rank,in], B [out,rank] BF16 (the working copies). A/B may be NULL (no
 * adapter); rank must then be 0, otherwise a multiple of 16. residual (may alias y) fuses the
 * following ops::add_inplace of the residual stream (qwen2.cu:126,150). Uses context scratch. */
int ta_lora_linear_fwd(ta_ctx* ctx, const void* x, const void* W, const void* bias, const void* A, const void* B,
                       const void* residual, void* y, int BT, int in_dim, int out_dim, int rank, float scale,
                       void* stream);
/* proj_bwd_x + AdapterModel::apply_lora_bwd (qwen2.cu:32-41; adapter_model.cu:131-220):
 *     dX[BT,in] = (accumulate_dx ? dX : 0) + dY.W + scale*(dY.B).A
 *     gA[rank,in] += scale*(dY.B)^T.x        gB[out,rank] += scale*dY^T.(x.A^T)        (FP32)
 * with h = x.A^T and dh = dY.B rounded to BF16 as in the reference. Uses context scratch (split-K
 * partials reduced in a fixed order, so results are bit-identical from run to run). */
int ta_lora_linear_bwd(ta_ctx* ctx, const void* x, const void* dY, const void* W, const void* A, const void* B, void* dX,
                       int accumulate_dx, float* gA, float* gB, int BT, int in_dim, int out_dim, int rank, float scale,
                       void* stream);

/* ── attention ─────────────────────────────────────────────────────────────────────────────
 * ops::sdpa_fwd / ops::sdpa_bwd (ops.hpp:52-70, src/backend/cuda/ops.cu:578-907): causal GQA
 * attention, scale 1/sqrt(head_dim), Q/out [B*T, Hq*hd], K/V [B*T, Hkv*hd]. Instead of the
 * reference's FP32 attn_w[B,Hq,T,T] cache only lse[B,Hq,T] (FP32, natural log) is kept, and the
 * backward also takes the forward output. head_dim 64 or 128. delta_scratch: FP32 [B*Hq*T] or NULL
 * (context scratch). */
int ta_flash_attn_fwd(ta_ctx* ctx, const void* Q, const void* K, const void* V, void* out, float* lse, int B, int T,
                      int Hq, int Hkv, int head_dim, void* stream);
int ta_flash_attn_bwd(ta_ctx* ctx, const void* dout, const void* Q, const void* K, const void* V, const void* out,
                      const float* lse, void* dQ, void* dK, void* dV, float* delta_scratch, int B, int T, int Hq, int Hkv,
                      int head_dim, void* stream);

/* ── optimiser ─────────────────────────────────────────────────────────────────────────────
 * ops::sum_sq_into (ops.hpp:154, ops.cu:1175-1193): *accum += sum g[i]^2, two-stage fixed-order. */
int ta_sum_sq_into(ta_ctx* ctx, const float* g, float* accum, long n, void* stream);
/* ops::adamw_step (ops.hpp:139-148, ops.cu:1139-1169); step is 1-based. */
int ta_adamw_step(ta_ctx* ctx, float* master, void* working, float* m, float* v, const float* grad, long n, float lr,
                  float beta1, float beta2, float eps, float weight_decay, int step, void* stream);
/* compute_grad_norm + clip_gradients + AdamW::step_all (src/trainer/adapt_trainer.cu:32-70,
 * src/trainer/adamw.cu:9-38) over ONE flat arena holding every LoRA tensor: norm = ||grad||_2; if
 * max_norm > 0 and norm > max_norm the gradient is scaled by max_norm/(norm+1e-6); then AdamW.
 * stats_dev (device, 2 floats) receives {norm, applied scale}; nothing is copied to the host.
 * scale_grads_in_place != 0 also leaves the scaled gradient in `grad`, as the reference does. */
int ta_gradnorm_clip_adamw(ta_ctx* ctx, float* master, void* working, float* m, float* v, float* grad, long n, float lr,
                           float beta1, float beta2, float eps, float weight_decay, int step, float max_norm,
                           float* stats_dev, int scale_grads_in_place, void* stream);

/* ── Centroid Accumulator ──────────────────────────────────────────────────────────────────
 * CentroidAccumulator::accumulate (include/tensor/centroid/centroid_accumulator.hpp:24-34,
 * src/centroid/centroid_accumulator.cpp:23-70) with the state (acc[D], weight) kept on the device.
 * hidden / grad_signal are BF16 [BT,D].
 *   TA_CENTROID_INTENDED  acc[d] += h[t,d]*||g[t,:]||_2, weight += ||g[t,:]||_2 (documented formula)
 *   TA_CENTROID_ASBUILT   what the shipped trainer computes (src/trainer/adapt_trainer.cu:210-232 hands
 *                         accumulate() FP32 copies which it re-reads as BF16): token u/2, half u%2 for
 *                         u < BT, gamma_u = ||g[tok, half*D/2 ..]||, acc[2m+1] += h[tok, half*D/2+m]*gamma_u */
#define TA_CENTROID_INTENDED 0
#define TA_CENTROID_ASBUILT  1
int ta_centroid_accumulate(ta_ctx* ctx, int mode, const void* hidden, const void* grad_signal, int BT, int D, float* acc,
                           float* weight, void* stream);
/* The k-means of CentroidAccumulator::merge_and_write (centroid_accumulator.cpp:114-157) on device
 * vectors [N,D] FP32: even-spread init, <= max_iters passes, strict '<' ties, early exit, zero
 * vectors for empty clusters; FP32 operation order kept so centres and assignments are bit-exact
 * with the host loop. centers [min(k,N), D] and assign [N] are device buffers; *k_out / *passes_out
 * are host ints. Synchronises the stream once per pass (to read the "changed" flag). */
int ta_kmeans_merge(ta_ctx* ctx, const float* vectors, int N, int D, int k, int max_iters, float* centers, int* assign,
                    int* k_out, int* passes_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TENSOR_ADAPT_B200_H */
