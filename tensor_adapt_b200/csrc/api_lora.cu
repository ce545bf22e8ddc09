// y = x.W^T (+bias) + s.(x.A^T).B^T and its backward, for one projection, through the C ABI.
//
// Forward: one skinny GEMM for h_s = bf16(s.x.A^T), then ONE segmented GEMM whose second K-segment
// (h_s, B) lands in the same TMEM accumulator as the base product - the rank-r path costs no extra
// pass over y.  Backward: dh_s = bf16(s.dY.B); dX = [beta.dX +] dY.W + dh_s.A as one two-segment GEMM;
// gB += dY^T.h_s and gA += dh_s^T.x as token-contracted split-K GEMMs with a fixed-order reduce.
// Folding s into h and dh keeps the reference's BF16 rounding points exactly when s is a power of two.
#include "lora.h"

namespace ta {

static inline size_t align256(size_t n) { return (n + 255) & ~size_t(255); }

int lora_down(ta_ctx* ctx, cudaStream_t s, const __nv_bfloat16* x, int BT, int in, const LoraRef& l, float scale,
              __nv_bfloat16* h_s) {
    GemmSegment g;
    g.A = x; g.lda = in; g.B = l.A; g.ldb = in; g.K = in;
    GemmOut o;
    o.C = h_s; o.ldc = l.r; o.alpha = scale;
    return seg_gemm(ctx, s, BT, l.r, &g, 1, o);
}

size_t lora_fwd_scratch_bytes(int BT, int r) { return align256(size_t(BT) * r * 2); }
size_t lora_bwd_scratch_bytes(const ta_ctx* ctx, int BT, int in, int out, int r) {
    return 2 * align256(size_t(BT) * r * 2) +
           align256(std::max(tokens_gemm_ws_bytes_max(ctx, out, r), tokens_gemm_ws_bytes_max(ctx, in, r)));
}

}  // namespace ta

using namespace ta;

extern "C" {

int ta_lora_linear_fwd(ta_ctx* ctx, const void* x, const void* W, const void* bias, const void* A, const void* B,
                       const void* residual, void* y, int BT, int in_dim, int out_dim, int rank, float scale,
                       void* stream) {
    if (!ctx || !x || !y || BT <= 0 || in_dim <= 0 || out_dim <= 0)
        return fail(ctx, TA_ERR_INVALID, "lora_linear_fwd: null argument or bad size");
    const bool lora = A && B && rank > 0;
    if (!W && !lora) return fail(ctx, TA_ERR_INVALID, "lora_linear_fwd: neither a base weight nor an adapter");
    if (lora && rank % 16 != 0) return fail(ctx, TA_ERR_UNSUPPORTED, "lora_linear_fwd: rank must be a multiple of 16");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    GemmSegment seg[2];
    int nseg = 0;
    if (W) {   // W == NULL: the adapter delta alone (AdapterModel::apply_lora_fwd on an existing projection output)
        seg[0].A = static_cast<const __nv_bfloat16*>(x); seg[0].lda = in_dim;
        seg[0].B = static_cast<const __nv_bfloat16*>(W); seg[0].ldb = in_dim; seg[0].K = in_dim;
        nseg = 1;
    }
    if (lora) {
        void* ws = nullptr;
        if (int rc = get_workspace(ctx, lora_fwd_scratch_bytes(BT, rank), &ws)) return rc;
        LoraRef l; l.A = static_cast<const __nv_bfloat16*>(A); l.B = static_cast<const __nv_bfloat16*>(B); l.r = rank;
        if (int rc = lora_down(ctx, s, static_cast<const __nv_bfloat16*>(x), BT, in_dim, l, scale, static_cast<__nv_bfloat16*>(ws))) return rc;
        GemmSegment& g = seg[nseg++];
        g.A = static_cast<const __nv_bfloat16*>(ws); g.lda = rank;
        g.B = l.B; g.ldb = rank; g.K = rank;
    }
    GemmOut o;
    o.C = y; o.ldc = out_dim;
    o.bias = static_cast<const __nv_bfloat16*>(bias);
    o.residual = static_cast<const __nv_bfloat16*>(residual);
    return seg_gemm(ctx, s, BT, out_dim, seg, nseg, o);
}

int ta_lora_linear_bwd(ta_ctx* ctx, const void* x, const void* dY, const void* W, const void* A, const void* B, void* dX,
                       int accumulate_dx, float* gA, float* gB, int BT, int in_dim, int out_dim, int rank, float scale,
                       void* stream) {
    if (!ctx || !dY || !dX || BT <= 0 || in_dim <= 0 || out_dim <= 0)
        return fail(ctx, TA_ERR_INVALID, "lora_linear_bwd: null argument or bad size");
    const bool lora = A && B && rank > 0;
    if (!W && !lora) return fail(ctx, TA_ERR_INVALID, "lora_linear_bwd: neither a base weight nor an adapter");
    if (lora && (!x || !gA || !gB)) return fail(ctx, TA_ERR_INVALID, "lora_linear_bwd: x, gA and gB are required with LoRA");
    if (lora && rank % 16 != 0) return fail(ctx, TA_ERR_UNSUPPORTED, "lora_linear_bwd: rank must be a multiple of 16");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const __nv_bfloat16* dy = static_cast<const __nv_bfloat16*>(dY);
    GemmSegment seg[2];
    int nseg = 0;
    if (W) {   // W == NULL: the adapter's share alone (AdapterModel::apply_lora_bwd)
        seg[0].A = dy; seg[0].lda = out_dim;
        seg[0].B = static_cast<const __nv_bfloat16*>(W); seg[0].ldb = in_dim; seg[0].b_mn = true; seg[0].K = out_dim;
        nseg = 1;
    }
    if (lora) {
        const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
        void* ws = nullptr;
        if (int rc = get_workspace(ctx, lora_bwd_scratch_bytes(ctx, BT, in_dim, out_dim, rank), &ws)) return rc;
        const size_t hb = align256(size_t(BT) * rank * 2);
        __nv_bfloat16* h_s = static_cast<__nv_bfloat16*>(ws);
        __nv_bfloat16* dh_s = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(ws) + hb);
        float* sk = reinterpret_cast<float*>(static_cast<char*>(ws) + 2 * hb);
        const size_t sk_bytes = ctx->ws_bytes - 2 * hb;
        LoraRef l; l.A = static_cast<const __nv_bfloat16*>(A); l.B = static_cast<const __nv_bfloat16*>(B); l.r = rank;
        // h_s = bf16(s.x.A^T)   (src/adapter/adapter_model.cu:142-152: recomputed in the backward)
        if (int rc = lora_down(ctx, s, xb, BT, in_dim, l, scale, h_s)) return rc;
        {   // dh_s = bf16(s.dY.B): B [out][r] read MN-major (k = out, n = r)   (:179-189)
            GemmSegment g; g.A = dy; g.lda = out_dim; g.B = l.B; g.ldb = rank; g.b_mn = true; g.K = out_dim;
            GemmOut o; o.C = dh_s; o.ldc = rank; o.alpha = scale;
            if (int rc = seg_gemm(ctx, s, BT, rank, &g, 1, o)) return rc;
        }
        {   // gB[out][r] += dY^T.h_s   (:155-176)
            GemmSegment g; g.A = dy; g.lda = out_dim; g.a_mn = true; g.B = h_s; g.ldb = rank; g.b_mn = true; g.K = BT;
            GemmOut o; o.C = gB; o.ldc = rank; o.f32 = true; o.accumulate = true;
            o.split_k = tokens_gemm_splits(ctx, out_dim, rank, BT); o.split_ws = sk; o.split_ws_bytes = sk_bytes;
            if (int rc = seg_gemm(ctx, s, out_dim, rank, &g, 1, o)) return rc;
        }
        {   // gA[r][in] += dh_s^T.x, computed as [in][r] tiles and stored transposed   (:190-207)
            GemmSegment g; g.A = xb; g.lda = in_dim; g.a_mn = true; g.B = dh_s; g.ldb = rank; g.b_mn = true; g.K = BT;
            GemmOut o; o.C = gA; o.ldc = in_dim; o.f32 = true; o.accumulate = true; o.transpose_out = true;
            o.split_k = tokens_gemm_splits(ctx, in_dim, rank, BT); o.split_ws = sk; o.split_ws_bytes = sk_bytes;
            if (int rc = seg_gemm(ctx, s, in_dim, rank, &g, 1, o)) return rc;
        }
        GemmSegment& g = seg[nseg++];
        g.A = dh_s; g.lda = rank; g.B = l.A; g.ldb = in_dim; g.b_mn = true; g.K = rank;
    }
    GemmOut o;
    o.C = dX; o.ldc = in_dim;
    if (accumulate_dx) o.residual = static_cast<const __nv_bfloat16*>(dX);
    return seg_gemm(ctx, s, BT, in_dim, seg, nseg, o);
}

}  // extern "C"
