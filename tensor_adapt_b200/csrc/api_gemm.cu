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

// logits = x.W^T, loss / dlogits, dx = dlogits.W for `chunk_rows` rows at a time: the [BT, V] logits of the
// reference (two 2.3 GiB tensors at 8 x 1024 tokens of a 152k vocabulary) shrink to one chunk buffer that
// the cross-entropy kernel overwrites in place with the gradient.
int ta_lmhead_ce_fwd_bwd(ta_ctx* ctx, const void* x, const void* lm_head, const int* targets, float* loss, void* dx, int BT, int H,
                         int V, float inv_count, void* logits_chunk, int chunk_rows, void* stream) {
    if (!ctx || !x || !lm_head || !targets || !loss || !dx || !logits_chunk || BT < 0 || H <= 0 || V <= 0 || chunk_rows <= 0)
        return fail(ctx, TA_ERR_INVALID, "lmhead_ce_fwd_bwd: null argument or bad size");
    const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
    __nv_bfloat16* dxb = static_cast<__nv_bfloat16*>(dx);
    for (int r0 = 0; r0 < BT; r0 += chunk_rows) {
        const int rows = BT - r0 < chunk_rows ? BT - r0 : chunk_rows;
        if (int rc = ta_gemm_bf16(ctx, rows, V, H, 1.f, xb + size_t(r0) * H, H, 0, lm_head, H, 0, nullptr, nullptr, logits_chunk, V, stream))
            return rc;
        if (int rc = ta_cross_entropy_fwd(ctx, logits_chunk, targets + r0, loss + r0, logits_chunk, rows, V, inv_count, stream)) return rc;
        if (int rc = ta_gemm_bf16(ctx, rows, H, V, 1.f, logits_chunk, V, 0, lm_head, H, 1, nullptr, nullptr, dxb + size_t(r0) * H, H, stream))
            return rc;
    }
    return TA_OK;
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
