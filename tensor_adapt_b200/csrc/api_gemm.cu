// C-ABI wrappers over the segmented-K tcgen05 GEMM for the two plain products of the path.
#include <algorithm>

#include "seg_gemm.h"

using namespace ta;

extern "C" {

int ta_gemm_bf16(ta_ctx* ctx, int M, int N, int K, float alpha, const void* A, long lda, int a_layout, const void* B,
                 long ldb, int b_layout, const void* bias, const void* residual, void* C, long ldc, void* stream) {
    if (!ctx) return TA_ERR_INVALID;
    GemmSegment s;
    s.A = static_cast<const __nv_bfloat16*>(A); s.lda = lda; s.a_mn = a_layout != 0;
    s.B = static_cast<const __nv_bfloat16*>(B); s.ldb = ldb; s.b_mn = b_layout != 0;
    s.K = K;
    GemmOut o;
    o.C = C; o.ldc = ldc; o.alpha = alpha;
    o.bias = static_cast<const __nv_bfloat16*>(bias);
    o.residual = static_cast<const __nv_bfloat16*>(residual);
    return seg_gemm(ctx, static_cast<cudaStream_t>(stream), M, N, &s, 1, o);
}

int ta_gemm_tokens_f32(ta_ctx* ctx, int M, int N, int K, float alpha, const void* A, long lda, const void* B, long ldb,
                       float* C, long ldc, int accumulate, int transpose_out, void* stream) {
    if (!ctx) return TA_ERR_INVALID;
    GemmSegment s;
    s.A = static_cast<const __nv_bfloat16*>(A); s.lda = lda; s.a_mn = true;
    s.B = static_cast<const __nv_bfloat16*>(B); s.ldb = ldb; s.b_mn = true;
    s.K = K;
    GemmOut o;
    o.C = C; o.ldc = ldc; o.alpha = alpha; o.f32 = true; o.accumulate = accumulate != 0;
    o.transpose_out = transpose_out != 0;
    o.split_k = tokens_gemm_splits(ctx, M, N, K);
    return seg_gemm(ctx, static_cast<cudaStream_t>(stream), M, N, &s, 1, o);
}

}  // extern "C"
