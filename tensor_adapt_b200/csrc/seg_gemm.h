// Segmented-K BF16 GEMM on tcgen05 / TMEM fed by TMA.
//
//   D[M,N] = alpha * sum_s  A_s[M,K_s] . B_s[N,K_s]^T   (+ bias[N]) (+ residual[M,N])
//
// Each segment names its own pair of operands, so a LoRA-augmented projection
// y = x.W^T + (s.h).B^T is ONE launch with two segments accumulating into the same TMEM tile, and
// the backward dX = dQ.Wq + dK.Wk + dV.Wv + dh_q.A_q + dh_k.A_k + dh_v.A_v is one launch with six.
// Operands may be K-major (element [row][k], k contiguous) or MN-major (element [k][row], row
// contiguous), which covers y = x.W^T (K-major W), dX = dY.W (MN-major W) and the token-contracted
// LoRA gradients (both operands MN-major) without transposed copies.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "ctx.h"

namespace ta {

constexpr int kMaxSegments = 6;

struct GemmSegment {
    const __nv_bfloat16* A = nullptr;   // K-major: [M][K] ; MN-major: [K][M]
    long lda = 0;                       // row pitch in elements
    bool a_mn = false;
    const __nv_bfloat16* B = nullptr;   // K-major: [N][K] ; MN-major: [K][N]
    long ldb = 0;
    bool b_mn = false;
    int K = 0;
    // fused gate/up ("dual") launches only: the up half's operand ([N][K] K-major, same pitch rules), and for a rank-r
    // segment the rank: A is then [M][2*k_half] = [h_gate | h_up], B / B2 are the two adapters' [N][k_half]
    const __nv_bfloat16* B2 = nullptr;
    long ldb2 = 0;
    int k_half = 0;
};

struct GemmOut {
    void* C = nullptr;                  // [M][ldc]  bf16 or fp32
    long ldc = 0;
    bool f32 = false;                   // output element type
    bool accumulate = false;            // fp32 only: C += result
    float alpha = 1.f;
    const __nv_bfloat16* bias = nullptr;      // [N] or null
    const __nv_bfloat16* residual = nullptr;  // [M][ldc] or null (may alias C)
    int split_k = 1;                    // >1: fp32 partials into ws[split][M][N] then a fixed-order reduce
    bool transpose_out = false;         // split-K reduce only: write C[n][m] (C is [N][ldc])
    float* split_ws = nullptr;          // split-K partials go here instead of the context workspace
    size_t split_ws_bytes = 0;
    bool no_host_state = false;         // encode tensor maps on the stack: no cache insert, no profiling events
    // Fused SwiGLU.  epi 1 ("dual" launch, every segment carries B2): N counts the GATE columns; a tile computes 128 gate
    // and the 128 matching up columns and stores gate -> C, up -> C2, act = silu(gate)*up -> C3 (all [M][ldc] BF16).
    // epi 2: the product is d_act; with the forward's gate_in / up_in it stores d_gate -> C and d_up -> C2 instead.
    int epi = 0;
    void* C2 = nullptr;
    void* C3 = nullptr;
    const __nv_bfloat16* gate_in = nullptr;
    const __nv_bfloat16* up_in = nullptr;
};

// Whether seg_gemm can run the fused SwiGLU forms for this many rows (they need the 256-row tile kernels).
bool seg_gemm_supports_swiglu(const ta_ctx* ctx, int M);
// Whether they are also the FASTER arrangement: true when the library's own choice for these launches is the CTA-pair
// kernel, whose epilogue runs under the next tile's main loop (16384 x 3584 x 18944: forward 2.98 ms against 3.17 ms for
// two GEMMs + silu_mul_fwd, backward 1.86 against 2.10 ms); on the single-CTA kernels the epilogue is exposed and the
// fused forms lose (3.63 / 2.38 ms).
bool seg_gemm_swiglu_pays(ta_ctx* ctx, int M);

// Split count the token-contracted gradient GEMM (M x N output, K tokens) should use, and the bytes
// of partials that many splits need.
int tokens_gemm_splits(const ta_ctx* ctx, int M, int N, int K);
size_t tokens_gemm_ws_bytes(const ta_ctx* ctx, int M, int N, int K);
size_t tokens_gemm_ws_bytes_max(const ta_ctx* ctx, int M, int N);   // for any token count

// Launches on `stream`; asynchronous. Returns TA_OK or a negative error code.
int seg_gemm(ta_ctx* ctx, cudaStream_t stream, int M, int N, const GemmSegment* segs, int nseg, const GemmOut& out);

}  // namespace ta
