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

// gate = x.Wg^T, up = x.Wu^T (each + its adapter) and act = silu(gate)*up in one launch (fused gate/up tiles).
int ta_swiglu_proj_fwd(ta_ctx* ctx, const void* x, const void* gate_w, const void* up_w, const void* A_gate_up, const void* B_gate,
                       const void* B_up, void* gate, void* up, void* act, int BT, int in_dim, int inter, int rank, float scale,
                       void* stream) {
    if (!ctx || !x || !gate_w || !up_w || !gate || !up || !act || BT <= 0 || in_dim <= 0 || inter <= 0)
        return fail(ctx, TA_ERR_INVALID, "swiglu_proj_fwd: null argument or bad size");
    const bool lora = A_gate_up && B_gate && B_up && rank > 0;
    if (lora && rank % 16) return fail(ctx, TA_ERR_UNSUPPORTED, "swiglu_proj_fwd: rank must be a multiple of 16");
    if (!seg_gemm_supports_swiglu(ctx, BT)) return fail(ctx, TA_ERR_UNSUPPORTED, "swiglu_proj_fwd: needs at least 256 rows");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
    GemmSegment seg[2];
    seg[0].A = xb; seg[0].lda = in_dim; seg[0].K = in_dim;
    seg[0].B = static_cast<const __nv_bfloat16*>(gate_w); seg[0].ldb = in_dim;
    seg[0].B2 = static_cast<const __nv_bfloat16*>(up_w); seg[0].ldb2 = in_dim;
    int nseg = 1;
    if (lora) {
        void* ws = nullptr;
        if (int rc = get_workspace(ctx, size_t(BT) * 2 * rank * 2 + 256, &ws)) return rc;
        GemmSegment g;   // h_s[BT][2r] = bf16(scale * x.[A_gate; A_up]^T): both adapters in one pass over x
        g.A = xb; g.lda = in_dim; g.B = static_cast<const __nv_bfloat16*>(A_gate_up); g.ldb = in_dim; g.K = in_dim;
        GemmOut ho; ho.C = ws; ho.ldc = 2 * rank; ho.alpha = scale;
        if (int rc = seg_gemm(ctx, s, BT, 2 * rank, &g, 1, ho)) return rc;
        seg[1].A = static_cast<const __nv_bfloat16*>(ws); seg[1].lda = 2 * rank; seg[1].K = 2 * rank; seg[1].k_half = rank;
        seg[1].B = static_cast<const __nv_bfloat16*>(B_gate); seg[1].ldb = rank;
        seg[1].B2 = static_cast<const __nv_bfloat16*>(B_up); seg[1].ldb2 = rank;
        nseg = 2;
    }
    GemmOut o;
    o.C = gate; o.C2 = up; o.C3 = act; o.ldc = inter; o.epi = 1;
    return seg_gemm(ctx, s, BT, inter, seg, nseg, o);
}

// d_act = dY.W_down (+ dh.A_down) turned into d_gate / d_up by the epilogue; d_act itself is never stored.
int ta_swiglu_down_bwd(ta_ctx* ctx, const void* dY, const void* down_w, const void* dh, const void* A_down, const void* gate,
                       const void* up, void* d_gate, void* d_up, int BT, int hidden, int inter, int rank, void* stream) {
    if (!ctx || !dY || !down_w || !gate || !up || !d_gate || !d_up || BT <= 0 || hidden <= 0 || inter <= 0)
        return fail(ctx, TA_ERR_INVALID, "swiglu_down_bwd: null argument or bad size");
    GemmSegment seg[2];
    seg[0].A = static_cast<const __nv_bfloat16*>(dY); seg[0].lda = hidden; seg[0].K = hidden;
    seg[0].B = static_cast<const __nv_bfloat16*>(down_w); seg[0].ldb = inter; seg[0].b_mn = true;
    int nseg = 1;
    if (dh && A_down && rank > 0) {
        if (rank % 16) return fail(ctx, TA_ERR_UNSUPPORTED, "swiglu_down_bwd: rank must be a multiple of 16");
        seg[1].A = static_cast<const __nv_bfloat16*>(dh); seg[1].lda = rank; seg[1].K = rank;
        seg[1].B = static_cast<const __nv_bfloat16*>(A_down); seg[1].ldb = inter; seg[1].b_mn = true;
        nseg = 2;
    }
    GemmOut o;
    o.C = d_gate; o.C2 = d_up; o.ldc = inter; o.epi = 2;
    o.gate_in = static_cast<const __nv_bfloat16*>(gate); o.up_in = static_cast<const __nv_bfloat16*>(up);
    return seg_gemm(ctx, static_cast<cudaStream_t>(stream), BT, inter, seg, nseg, o);
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
