/* tensor_adapt_b200 - C ABI of the B200-native LoRA training hot path.
 *
 * Drop-in boundary for carbon-os/tensor-adapt's CUDA backend and trainer: every entry point
 * below names the reference interface it replaces (file:line inside the reference tree).  The
 * reference has no FFI layer of its own; its boundary is the C++ API in include/tensor/, so each
 * function here is what a thin C++ shim with the reference's name and signature calls (the shim
 * sources under shim/ implement the reference's own headers that way).
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
/* Self-test of the bounded device waits (no counterpart in the reference, whose kernels never wait on one
 * another): a one-warp kernel waits limit_us microseconds on a barrier that nothing arrives at, gives up, records
 * its status code and returns.  Afterwards ta_device_status() reports TA_ERR_DEVICE_TIMEOUT with *status = 106 and
 * the context is usable as before.  *wait_returned_true receives 0 (the wait gave up), *abort_flag_seen 1 (the
 * rest of the CTA saw the abort flag).  Synchronises the stream. */
int ta_selftest_bounded_wait(ta_ctx* ctx, int limit_us, int* wait_returned_true, int* abort_flag_seen, void* stream);
/* Kernels launched through this context so far. */
long ta_launch_count(const ta_ctx* ctx);
/* Experiment knob, no counterpart in the reference: force the GEMM tile (tile_n in {64,128,224,256},
 * tile_m_halves 1 = 128-row or 2 = 256-row tiles; 0,0 = the built-in cost model) and / or select a
 * kernel for 256-wide tiles (cta_pair 0: the library's choice - the 256 x 256 CTA-pair kernel of mode 3 where the device
 * can keep a pair resident on every two SMs; -1: single-CTA kernels only; 1: 512 x 256 pair tiles; 2: 256 x 256 pair tiles
 * with double-buffered accumulators; 3: as 2 with 128-wide k blocks).  Results are bit-identical for every choice.
 * Threading: a context, and every object created from it, belongs to ONE host thread at a time (the
 * reference's Device is single-threaded too); the library keeps per-device launch attributes and the
 * static-scratch address in unsynchronised process-wide state that is written on first use. */
int ta_ctx_set_gemm_tuning(ta_ctx* ctx, int tile_n, int tile_m_halves, int cta_pair);
/* Experiment knob, no counterpart in the reference: the order in which the persistent CTAs walk the output tiles
 * (which operand panels a wave shares through L2): row groups of group_m tiles, inside column bands of group_n tiles
 * (0, 0 = the built-in choice).  Results are identical for every order; only DRAM traffic and speed change. */
int ta_ctx_set_gemm_raster(ta_ctx* ctx, int group_m, int group_n);
/* Optional CUDA-event timing of the tensor-core kernels, off by default (it adds two event records
 * per launch). Classes: 0 = segmented GEMM with tiles >= 128 wide, 1 = skinny GEMMs (rank-r and
 * split-K), 2 = attention forward, 3 = attention backward. ta_profile_read synchronises the device
 * and returns, per class, launches, algorithmic FLOPs and summed device milliseconds since the last
 * read. No counterpart in the reference (it has no profiling hooks). */
int ta_profile_enable(ta_ctx* ctx, int on);
int ta_profile_read(ta_ctx* ctx, int n_classes, long* launches, double* work, double* ms);

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
/* The head of Qwen2Base::forward + the loss + the head of Qwen2Base::backward in one call
 * (src/base/arch/qwen2.cu:163-175 lm_head GEMM, src/backend/cuda/ops.cu:958-1020 cross_entropy_fwd,
 * qwen2.cu:203-205 dres = dlogits.W): x [BT,H] BF16 (final-norm output), lm_head [V,H] BF16, targets
 * [BT], loss [BT] FP32, dx [BT,H] BF16. Rows are processed chunk_rows at a time through
 * logits_chunk [chunk_rows, V] BF16 (caller-provided device scratch), so no [BT,V] tensor exists;
 * results are identical to running the three reference calls on the whole batch. */
int ta_lmhead_ce_fwd_bwd(ta_ctx* ctx, const void* x, const void* lm_head, const int* targets, float* loss, void* dx, int BT, int H,
                         int V, float inv_count, void* logits_chunk, int chunk_rows, void* stream);
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
/* The same product for callers that cannot allocate device memory (a host application that owns all of
 * device memory through its own pool, a plugin sandbox that forbids cudaMalloc and the device-wide
 * synchronisation it implies).  It has no counterpart in the reference,
 * whose every op allocates its temporaries (src/adapter/adapter_model.cu:142-191).  Same arguments and
 * results as ta_gemm_tokens_f32, but the split-K partials live in a fixed array inside the library image
 * (TA_STATIC_SCRATCH_BYTES, held by every GPU that loads the library until exit) and the call performs no
 * cudaMalloc/cudaFree and inserts nothing into the tensor-map cache.
 *   - sizes whose partials (splits * M * N * 4 bytes) exceed TA_STATIC_SCRATCH_BYTES are rejected with
 *     TA_ERR_NOMEM and a message naming the sizes; use ta_gemm_tokens_f32 for those;
 *   - the context's device must be the current device; the FIRST call on a device resolves the array's
 *     device address (cudaGetSymbolAddress) - make that first call before any stream capture begins;
 *   - all calls share the one array: calls that may overlap on the GPU (different streams) race on it and
 *     must be serialised by the caller. */
#define TA_STATIC_SCRATCH_BYTES (8u << 20)
int ta_gemm_tokens_f32_static(ta_ctx* ctx, int M, int N, int K, float alpha, const void* A, long lda, const void* B,
                              long ldb, float* C, long ldc, int accumulate, int transpose_out, void* stream);

/* ── LoRA-augmented projection ─────────────────────────────────────────────────────────────
 * proj_fwd + ops::add_bias + AdapterModel::apply_lora_fwd (src/base/arch/qwen2.cu:21-30,95-108;
 * src/adapter/adapter_model.cu:96-129) as one fused product:
 *     y[BT,out] = x.W^T (+ bias) + scale*(x.A^T).B^T (+ residual)
 * x [BT,in], W [out,in], A [rank,in], B [out,rank] BF16 (the working copies). A/B may be NULL (no
 * adapter); rank must then be 0, otherwise a multiple of 16. residual (may alias y) fuses the
 * following ops::add_inplace of the residual stream (qwen2.cu:126,150). W may be NULL: only the adapter
 * delta is formed, y = residual + scale*(x.A^T).B^T, which with residual == y is
 * AdapterModel::apply_lora_fwd on an existing projection output. Uses context scratch. */
int ta_lora_linear_fwd(ta_ctx* ctx, const void* x, const void* W, const void* bias, const void* A, const void* B,
                       const void* residual, void* y, int BT, int in_dim, int out_dim, int rank, float scale,
                       void* stream);
/* proj_bwd_x + AdapterModel::apply_lora_bwd (qwen2.cu:32-41; adapter_model.cu:131-220):
 *     dX[BT,in] = (accumulate_dx ? dX : 0) + dY.W + scale*(dY.B).A
 *     gA[rank,in] += scale*(dY.B)^T.x        gB[out,rank] += scale*dY^T.(x.A^T)        (FP32)
 * with h = x.A^T and dh = dY.B rounded to BF16 as in the reference. W may be NULL (the dY.W term is
 * left out: AdapterModel::apply_lora_bwd with accumulate_dx = 1). Uses context scratch (split-K
 * partials reduced in a fixed order, so results are bit-identical from run to run). */
int ta_lora_linear_bwd(ta_ctx* ctx, const void* x, const void* dY, const void* W, const void* A, const void* B, void* dX,
                       int accumulate_dx, float* gA, float* gB, int BT, int in_dim, int out_dim, int rank, float scale,
                       void* stream);

/* proj_fwd x 2 + apply_lora_fwd x 2 + ops::silu_mul_fwd of the MLP (src/base/arch/qwen2.cu:137-147,
 * src/backend/cuda/ops.cu:913-923) as one launch: every tile holds 128 gate columns and the 128 matching up columns,
 * and the epilogue stores gate, up (both needed by the backward) and act = silu(gate) * up.
 *     gate = x.gate_w^T + scale*(x.A_gate^T).B_gate^T      up likewise      act[BT, inter]
 * A_gate_up is the two adapters' A blocks back to back, [2*rank][in_dim] (NULL: no adapters); rank % 16 == 0; BT >= 256. */
int ta_swiglu_proj_fwd(ta_ctx* ctx, const void* x, const void* gate_w, const void* up_w, const void* A_gate_up, const void* B_gate,
                       const void* B_up, void* gate, void* up, void* act, int BT, int in_dim, int inter, int rank, float scale,
                       void* stream);
/* proj_bwd_x of the down projection (+ the dX share of apply_lora_bwd) + ops::silu_mul_bwd (qwen2.cu:221-230,
 * ops.cu:925-941) as one launch: d_act = dY.down_w (+ dh.A_down) stays in tensor memory and the epilogue writes
 *     d_gate = d_act * up * silu'(gate)      d_up = d_act * silu(gate)
 * dY [BT, hidden], down_w [hidden, inter], dh [BT, rank] = bf16(scale*dY.B_down) or NULL, A_down [rank, inter]. */
int ta_swiglu_down_bwd(ta_ctx* ctx, const void* dY, const void* down_w, const void* dh, const void* A_down, const void* gate,
                       const void* up, void* d_gate, void* d_up, int BT, int hidden, int inter, int rank, void* stream);

/* ── attention ─────────────────────────────────────────────────────────────────────────────
 * ops::sdpa_fwd / ops::sdpa_bwd (ops.hpp:52-70, src/backend/cuda/ops.cu:578-907): causal GQA
 * attention, scale 1/sqrt(head_dim), Q/out [B*T, Hq*hd], K/V [B*T, Hkv*hd]. Instead of the
 * reference's FP32 attn_w[B,Hq,T,T] cache only lse[B,Hq,T] (FP32, natural log) is kept, and the
 * backward also takes the forward output. head_dim 64 or 128. delta_scratch: FP32 [B*Hq*T] or NULL
 * (context scratch).  A backward call with fewer than two (128-key tile, KV head, batch) triples per SM shares a
 * group's query heads out over several CTAs and keeps their FP32 partial dK / dV sums in the context scratch as well
 * (2 * parts * B*T*Hkv*hd floats, parts <= Hq/Hkv; the scratch grows on first use); results are bit-reproducible. */
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
/* The merge the README describes (README.md:73-79) but the reference does not implement: seeded
 * k-means++ start (init_mode TA_KMEANS_INIT_PLUSPLUS: 64-bit LCG draws, FP32 distances in the order
 * above, FP64 running sums for the pick - reproducible bit for bit) or the reference's even-spread
 * start (TA_KMEANS_INIT_EVEN), the same Lloyd passes, then - if rank_by_mass - clusters reordered by
 * descending summed gradient mass (mass [N] device FP32, NULL = count; FP64 sums, ties keep index
 * order): centers and assign come back in ranked order / labels, cluster_mass [k] (device FP64, may be
 * NULL) holds the masses, init_index [k] (device, may be NULL) the chosen start vectors. No
 * reference counterpart. */
#define TA_KMEANS_INIT_EVEN     0
#define TA_KMEANS_INIT_PLUSPLUS 1
int ta_kmeans_merge_ex(ta_ctx* ctx, const float* vectors, const float* mass, int N, int D, int k, int max_iters, int init_mode,
                       unsigned long long seed, int rank_by_mass, float* centers, int* assign, double* cluster_mass,
                       int* init_index, int* k_out, int* passes_out, void* stream);

/* ── model / adapter / trainer ─────────────────────────────────────────────────────────────
 * The trainer object stands where the reference has FrozenBase + AdapterModel + AdamW +
 * CentroidAccumulator + AdaptTrainer::Impl (include/tensor/base/frozen_base.hpp:15-56,
 * include/tensor/adapter/adapter_model.hpp:26-95, include/tensor/trainer/adapt_trainer.hpp:18-78,
 * src/trainer/adapt_trainer.cu:96-277).  All device memory is allocated once at creation. */
typedef struct ta_model_config {      /* BaseConfig, frozen_base.hpp:15-29 */
    int vocab, hidden, layers, q_heads, kv_heads, head_dim, intermediate;
    float rms_eps, rope_theta;
    int tie_embeddings;
} ta_model_config;

#define TA_TARGET_Q    1
#define TA_TARGET_K    2
#define TA_TARGET_V    4
#define TA_TARGET_O    8
#define TA_TARGET_GATE 16             /* gate/up/down adapters are an extension: the reference wires */
#define TA_TARGET_UP   32             /* q/k/v/o only (src/adapter/adapter_model.cu:82-87)           */
#define TA_TARGET_DOWN 64
#define TA_TARGETS_QKVO 15
#define TA_TARGETS_ALL  127

typedef struct ta_adapter_config {    /* AdapterConfig, include/tensor/adapter/adapter_config.hpp:25-70 */
    int rank;
    float alpha;                      /* effective scale = alpha / rank */
    int targets;                      /* TA_TARGET_* bit mask */
    float lr, grad_clip;
    int warmup_steps;
    float beta1, beta2, eps, weight_decay;
    int centroid_modes;               /* bit 0: intended accumulator, bit 1: as-built accumulator,
                                         bit 2: per-layer bank (one intended accumulator per layer) */
} ta_adapter_config;

typedef struct ta_step_metrics {      /* StepMetrics, adapt_trainer.hpp:18-27 (wall-clock fields are the caller's) */
    long step, tokens_consumed;
    float loss;                       /* mean over per-token losses > 1e-9 (adapt_trainer.cu:237-246) */
    float learning_rate;
    float grad_norm;                  /* min(norm, grad_clip), as the reference reports (adapt_trainer.cu:250) */
    float grad_norm_raw;
} ta_step_metrics;

typedef struct ta_trainer ta_trainer;

/* AdaptTrainer::create (adapt_trainer.cu:280-286) + AdapterModel::create (adapter_model.cu:69-90):
 * allocates the frozen-base arena, the flat LoRA arrays (FP32 master / m / v / grad + BF16 working)
 * and an activation arena for micro-batches of `micro_batch` sequences of `seq_len` tokens.
 * A is initialised with the reference's hash-Kaiming values and B with zeros; base weights are left
 * uninitialised until ta_trainer_init_random() or uploads through ta_trainer_tensor(). */
int ta_trainer_create(ta_ctx* ctx, const ta_model_config* model, const ta_adapter_config* adapter, int micro_batch,
                      int seq_len, void* stream, ta_trainer** out);
int ta_trainer_destroy(ta_trainer* tr);
/* Random-init frozen base on the device: matrices and biases ~N(0, std), norm weights 1 (the
 * reference loads these from safetensors, src/base/base_loader.cpp:112-166; synthetic here). */
int ta_trainer_init_random(ta_trainer* tr, unsigned long long seed, float std);
/* Device pointer and shape of a named tensor, for uploads / read-backs with cudaMemcpy:
 *   "embed" "final_norm" "lm_head" "l<i>.{input_norm,post_norm,q_w,k_w,v_w,o_w,q_b,k_b,v_b,gate_w,up_w,down_w}"
 *   "l<i>.lora.<q|k|v|o|gate|up|down>.<A|B|gA|gB|mA|mB|vA|vB|A_bf16|B_bf16>"
 *   "lora.master" "lora.grad" "lora.m" "lora.v" "lora.working" (whole flat arrays)
 *   "centroid.acc" "centroid.weight" "centroid_asbuilt.acc" "centroid_asbuilt.weight"
 *   "centroid_bank.acc" [layers, hidden] "centroid_bank.weight" [layers]
 *   "l<i>.cache.<x_normed|Q|K|V|attn_out|r_in|r_mid>" "cache.dx_attn_in" (last micro-batch, layer 0)
 * dtype: 0 = FP32, 1 = BF16. pitch is the row pitch in elements. */
int ta_trainer_tensor(ta_trainer* tr, const char* name, void** dev_ptr, long* rows, long* cols, long* pitch, int* dtype);
/* Switches of the step's fusions, for A/B comparisons: "fuse_swiglu" (1: SwiGLU forward / backward run inside the
 * gate-up and down-dX GEMM epilogues; 0: separate silu_mul kernels as the reference has them; -1, the default: fused
 * where the CTA-pair GEMM kernel carries those launches and hides the epilogue, separate otherwise).  The forward is
 * bit-identical either way; the fused backward skips one BF16 rounding of d_act.  No reference counterpart. */
int ta_trainer_set_option(ta_trainer* tr, const char* name, int value);
/* Re-derive the BF16 working copies from the FP32 masters (after masters were uploaded). */
int ta_trainer_sync_working(ta_trainer* tr);
/* AdapterModel::zero_grad (adapter_model.cu:222-229): one memset of the flat gradient array. */
int ta_trainer_zero_grad(ta_trainer* tr);
/* Steps 3-7 of do_step (adapt_trainer.cu:190-232) for `B` sequences of `T` tokens: zero_grad is NOT
 * included (call ta_trainer_zero_grad once per optimiser step), so several calls accumulate.
 * tokens / targets: B*T int32, HOST memory when host_inputs != 0 (copied H2D inside), else device.
 * The batch is processed in micro-batches; the cross-entropy gradient is scaled by 1/global_tokens
 * (pass B*T for a single GPU; the data-parallel caller passes the global count and then sum-reduces
 * "lora.grad"). Centroid accumulation (per layer: hidden = post-input-norm activations, signal =
 * d loss / d those activations, adapt_trainer.cu:210-232) runs on the device in the configured modes. */
int ta_trainer_forward_backward(ta_trainer* tr, const int* tokens, const int* targets, int B, int T, long global_tokens,
                                int host_inputs);
/* compute_grad_norm + clip_gradients + AdamW::step_all (adapt_trainer.cu:248-253) then one D2H copy
 * of {norm, loss sum, loss count}; fills *out. lr < 0 selects CosineSchedule::lr_at(step)
 * (cosine_schedule.hpp:18-29) with total_steps given. Synchronises the stream. */
int ta_trainer_optimizer_step(ta_trainer* tr, float lr, long total_steps, ta_step_metrics* out);
/* AdaptTrainer::step (adapt_trainer.cu:130-277) on caller-provided ids: zero_grad + forward_backward +
 * optimizer_step. */
int ta_trainer_step(ta_trainer* tr, const int* tokens, const int* targets, int B, int T, float lr, long total_steps,
                    int host_inputs, ta_step_metrics* out);
/* CentroidAccumulator::write_snapshot (src/centroid/centroid_accumulator.cpp:72-91): normalised
 * centroid acc/weight of the chosen mode (0 intended, 1 as-built) to `path` (may be NULL) in the
 * reference's layout int32 D | D x f32 | f32 weight, and into centroid_out[D] / weight_out (host, may be
 * NULL). Returns TA_OK without writing when the weight is zero, as the reference does. */
int ta_trainer_write_snapshot(ta_trainer* tr, int mode, const char* path, float* centroid_out, float* weight_out);
/* Multi-vector snapshot ("bank"): one normalised centroid per layer (centroid_modes bit 2), written as the
 * reference's snapshot record int32 D | D x f32 | f32 weight repeated per layer, so a one-layer bank is exactly a
 * reference snapshot file and the reference's reader sees the first record of a longer one.  centroids_out
 * [layers*D] / weights_out [layers] (host, may be NULL); *n_records = layers with non-zero weight.  The README's
 * "bank of vectors per snapshot" (README.md:73-79) has no code in the reference: no counterpart.
 * ta_centroid_merge_dir_ex clusters every record of every file. */
int ta_trainer_write_snapshot_bank(ta_trainer* tr, const char* path, float* centroids_out, float* weights_out, int* n_records);
/* AdapterWriter::save_checkpoint / save_final (src/checkpoint/adapter_writer.cpp:130-159): writes
 * adapter.safetensors (BF16 of the FP32 masters, flat shapes, reference tensor names), adapter.json
 * and, unless final != 0, train_state.json into `dir`, byte-compatible with the reference's files. */
int ta_trainer_save_checkpoint(ta_trainer* tr, const char* dir, const char* domain, long step, long tokens, int final_);
/* "architecture" and "base_sha" written into adapter.json (BaseConfig::arch_name / base_sha). */
int ta_trainer_set_meta(ta_trainer* tr, const char* arch_name, const char* base_sha);
/* CentroidAccumulator::merge_and_write on the in-memory, chronological snapshot list
 * (centroid_accumulator.cpp:93-168 as called from AdaptTrainer::save_adapter, adapt_trainer.cu:322-325). */
int ta_trainer_merge_snapshots(ta_trainer* tr, int k, const char* out_path, int* passes);

/* ── data-parallel exchange ────────────────────────────────────────────────────────────────
 * The reference has no multi-GPU code; nothing here replaces a reference interface.  One process per GPU; every
 * rank holds the frozen base and the LoRA state, takes its shard of the global batch, scales its cross-entropy
 * gradient by 1/global_tokens (ta_trainer_forward_backward) and the flat FP32 gradient array is SUM-reduced with
 * NCCL, together with the (loss sum, loss count) pair, before the replicated optimiser step.  NCCL is loaded at
 * run time (the copy already in the process, else libnccl.so.2); without it these calls return
 * TA_ERR_UNSUPPORTED and everything else works. */
typedef struct ta_comm ta_comm;
/* ncclGetUniqueId: rank 0 fills `out` (>= 128 bytes) and hands the bytes to the other ranks by any host channel. */
int ta_comm_unique_id(void* out, size_t bytes);
/* ncclCommInitRank on the context's device, plus the side stream the exchange runs on. Collective: every rank calls it. */
int ta_comm_create(ta_ctx* ctx, int rank, int world, const void* unique_id, size_t bytes, ta_comm** out);
int ta_comm_destroy(ta_comm* comm);
int ta_comm_info(const ta_comm* comm, int* rank, int* world);
/* One in-place all-reduce of "lora.grad" and of step.stats[2:4], ordered after the trainer's stream and awaited by
 * it: call between ta_trainer_forward_backward and ta_trainer_optimizer_step. */
int ta_allreduce_grads(ta_trainer* tr, ta_comm* comm);
/* Attach (or with NULL detach) a communicator: ta_trainer_forward_backward then performs the exchange itself,
 * bucketed per layer - the slice of a layer is all-reduced on the communicator's stream as soon as that layer's
 * backward has been issued in the LAST micro-batch of the call, overlapping the transfer with the remaining
 * layers - and the trainer's stream waits for the last bucket.  Requires ONE forward_backward call per optimiser
 * step (the call's micro-batches accumulate; a second call would add to already-reduced gradients). */
int ta_trainer_set_comm(ta_trainer* tr, ta_comm* comm);

/* ── real weights and resume ─────────────────────────────────────────────────────────────── */
/* parser::ModelConfig::from_dir + the derived fields of base::BaseLoader::load
 * (src/parser/config.cpp:43-110,132-134; src/base/base_loader.cpp:90-110,160): reads <dir>/config.json with
 * the reference's defaults, head_dim = hidden / heads, tie_embeddings = the shards hold no
 * "lm_head.weight"; arch_name = "model_type"; sha_hex = SHA-256 of the "name:size;" listing of the
 * directory's *.safetensors files sorted by name (base_loader.cpp:30-52). Host only, no GPU needed.
 * TA_ERR_IO (unreadable / malformed files, text in err_text) or TA_ERR_UNSUPPORTED (architecture
 * neither qwen* nor llama*, after applying arch_hint like detect_arch, base_loader.cpp:21-28). */
int ta_base_probe(const char* dir, const char* arch_hint, ta_model_config* mc, char* arch_name, int arch_cap, char* sha_hex,
                  int sha_cap, char* err_text, int err_cap);
/* base::BaseLoader::load (src/base/base_loader.cpp:80-170) into the trainer's weight arena: shard
 * discovery as parser::WeightMap::open (src/parser/weight_map.cpp:26-68: a .safetensors file, else
 * <dir>/model.safetensors alone, else every *.safetensors by name), header validation as
 * parser::SafeTensors (src/parser/safetensors.cpp:86-226), Hugging Face tensor names, BF16 copied as is,
 * F32 rounded to BF16 (RNE), any other dtype refused (TA_ERR_UNSUPPORTED) like upload_bf16
 * (base_loader.cpp:54-74). Unlike the reference, element counts are checked against the config. Also
 * sets the architecture / base_sha that adapter.json records. */
int ta_trainer_load_base(ta_trainer* tr, const char* dir, const char* arch_hint);
/* Writes <dir>/optimizer.safetensors: FP32 masters, AdamW m and v (the flat arrays), both centroid
 * accumulators, step and tokens_consumed. The reference documents this file (README.md:569-582) but has
 * no code for it: no reference counterpart. */
int ta_trainer_save_optimizer(ta_trainer* tr, const char* dir);
/* Resume (README.md:646-661; absent from the reference's code): validates <dir>/adapter.json (rank,
 * alpha, base_sha) against this trainer, then restores masters / moments / centroid sums / step / tokens
 * from optimizer.safetensors, or - for a checkpoint the reference wrote - masters from the BF16
 * adapter.safetensors with zero moments and step / tokens from train_state.json. */
int ta_trainer_resume(ta_trainer* tr, const char* dir);
/* Optimiser steps taken and tokens consumed so far (StepMetrics::step / tokens_consumed,
 * include/tensor/trainer/adapt_trainer.hpp), e.g. after ta_trainer_resume. */
int ta_trainer_counters(ta_trainer* tr, long* step, long* tokens_consumed);

/* ── token stream in HBM ─────────────────────────────────────────────────────────────────── */
typedef struct ta_dataset ta_dataset;
/* data::Dataset::load (src/data/dataset.cpp:15-53): a .bin file or a directory of .bin files (sorted by
 * path) of 32-bit token ids, concatenated - here into device memory, once. */
int ta_dataset_load(ta_ctx* ctx, const char* path, ta_dataset** out);
int ta_dataset_destroy(ta_dataset* ds);
/* Dataset::total_tokens / tokens_consumed and the read position (include/tensor/data/dataset.hpp). */
int ta_dataset_info(const ta_dataset* ds, long* total_tokens, long* position, long* tokens_consumed);
/* Restores the read position on resume (README.md:646-661 "continues ... same data position"); no
 * reference code. */
int ta_dataset_seek(ta_dataset* ds, long position, long tokens_consumed);
/* Dataset::next_batch (src/data/dataset.cpp:55-71) on the device: B windows of T tokens from the read
 * position with wrap-around, targets = the next token; the position advances by B*T. Only sequences
 * [first_seq, first_seq + n_seq) are materialised (a data-parallel rank's shard of the global batch)
 * into ids_dev / targets_dev [n_seq*T]. mask != 0 also applies the assistant-only target masking of
 * src/trainer/adapt_trainer.cu:145-182 in the same kernel. */
int ta_dataset_next_batch(ta_dataset* ds, int B, int T, int first_seq, int n_seq, int* ids_dev, int* targets_dev, int mask,
                          void* stream);
/* The masking alone (src/trainer/adapt_trainer.cu:145-182) on device arrays; ta_mask_targets is the host form. */
int ta_mask_targets_device(ta_ctx* ctx, const int* input_ids, int* target_ids, int B, int T, void* stream);
/* AdaptTrainer::step as the reference runs it (do_step, src/trainer/adapt_trainer.cu:130-277: next_batch,
 * masking, zero_grad, forward, loss, backward, centroid, clip, AdamW) with the batch drawn on the device. */
int ta_trainer_step_dataset(ta_trainer* tr, ta_dataset* ds, int B, int mask, float lr, long total_steps, ta_step_metrics* out);

/* ── host-side logic mirrored from the reference ─────────────────────────────────────────── */
/* CosineSchedule::lr_at (include/tensor/trainer/cosine_schedule.hpp:18-29). */
float ta_cosine_lr(float base_lr, long warmup_steps, long total_steps, long step, float floor_frac);
/* Assistant-only target masking (src/trainer/adapt_trainer.cu:145-182), in place on host arrays. */
void ta_mask_targets(const int* input_ids, int* target_ids, int B, int T);
/* k_kaiming_init_f32 (src/adapter/adapter_model.cu:28-39) on the host: out[rank*in_dim]. */
void ta_kaiming_init_host(float* out, int in_dim, int rank, unsigned seed);
/* CentroidMerge::run (src/centroid/centroid_merge.cpp:12-31): reads every *.centroid in `dir` (in
 * directory-iteration order, as the reference does), clusters on the GPU with ta_kmeans_merge and
 * writes int32 k | int32 D | k*D f32 to out_path. *n_vectors / *passes (may be NULL) report what ran. */
int ta_centroid_merge_dir(ta_ctx* ctx, const char* dir, const char* out_path, int k, int* n_vectors, int* passes);
/* The same over ta_kmeans_merge_ex: seeded k-means++ start and / or the bank ordered by gradient mass,
 * the mass of a snapshot being the trailing weight field of its record (README.md:73-79 "merged cluster
 * bank, gradient-ranked"); files that hold several records (snapshot banks) contribute all of them, in file
 * order; same output layout. No reference counterpart. */
int ta_centroid_merge_dir_ex(ta_ctx* ctx, const char* dir, const char* out_path, int k, int init_mode, unsigned long long seed,
                             int rank_by_mass, int* n_vectors, int* passes);
/* Host <-> device copies for callers without a CUDA runtime binding (synchronous). */
int ta_memcpy_h2d(void* dst_dev, const void* src_host, size_t bytes);
int ta_memcpy_d2h(void* dst_host, const void* src_dev, size_t bytes);

#ifdef __cplusplus
}
#endif
#endif /* TENSOR_ADAPT_B200_H */
