// Training-step orchestration: Qwen2 forward / backward over the fused kernels, cross-entropy,
// centroid accumulation, gradient norm / clip / AdamW.  One stream, no allocation and no host
// synchronisation inside forward_backward; the optimiser step ends with a single small D2H copy.
//
// Op order and rounding points follow Qwen2Base::forward / backward (src/base/arch/qwen2.cu:47-308)
// with these fusions: bias + LoRA delta + residual add in the GEMM epilogue (one BF16 rounding where
// the reference rounds up to four times), q/k/v (and gate/up) input gradients summed in one TMEM
// accumulator, rms_norm_bwd + residual-gradient add, attention without the [T,T] cache.
#include "trainer.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>

#include "ptx.cuh"

namespace ta {

const char* const kTargetNames[T_COUNT] = {"q", "k", "v", "o", "gate", "up", "down"};

namespace {

using bf16 = __nv_bfloat16;

// ── device helpers ──────────────────────────────────────────────────────────

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull; z ^= z >> 27; z *= 0x94D049BB133111EBull; z ^= z >> 31;
    return z;
}
// Approximately normal N(0, stdv) BF16 values from an integer hash: the centred sum of twelve 16-bit fields of
// three 64-bit hashes (variance 65536^2 - 1), scaled with single correctly-rounded operations only, so any
// compiler setting (fast-math included) produces the same bits - the parity harness that drives the reference
// fills its weights with the same function.
__global__ void fill_normal_kernel(bf16* p, long n, float stdv, unsigned long long seed) {
    const float c = __fmul_rn(stdv, 1.52587890625e-05f);   // stdv / 65536, exact
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < n; i += long(gridDim.x) * blockDim.x) {
        const unsigned long long x = (unsigned long long)(i + 1) * 0x9E3779B97F4A7C15ull + seed * 0xD1B54A32D192ED03ull;
        const unsigned long long z[3] = {mix64(x), mix64(x ^ 0xA5A5A5A5A5A5A5A5ull), mix64(x + 0x632BE59BD9B4E019ull)};
        int sum = 0;
#pragma unroll
        for (int k = 0; k < 3; k++)
            sum += int(z[k] & 0xFFFF) + int((z[k] >> 16) & 0xFFFF) + int((z[k] >> 32) & 0xFFFF) + int(z[k] >> 48);
        p[i] = __float2bfloat16_rn(__fmul_rn(__int2float_rn(sum - 6 * 65535), c));
    }
}
__global__ void fill_const_kernel(bf16* p, long n, float v) {
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < n; i += long(gridDim.x) * blockDim.x)
        p[i] = __float2bfloat16(v);
}
// Integer-hash uniform in [-1,1] * sqrt(1/in_dim): the values k_kaiming_init_f32 produces
// (src/adapter/adapter_model.cu:28-39), written for the logical [rank][in_dim] block.
__host__ __device__ inline float kaiming_value(unsigned i, int in_dim, unsigned seed) {
    unsigned r = seed ^ (i * 2654435761u);
    r = r ^ (r >> 16); r *= 0x45d9f3bu; r ^= (r >> 16);
    const float u = float(r & 0xFFFFFFu) / float(0xFFFFFF) * 2.f - 1.f;
#ifdef __CUDA_ARCH__
    return u * sqrtf(1.f / float(in_dim));
#else
    return u * std::sqrt(1.f / float(in_dim));
#endif
}
__global__ void kaiming_kernel(float* A, int in_dim, int rank, unsigned seed) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < in_dim * rank) A[i] = kaiming_value(unsigned(i), in_dim, seed);
}
// stats[2] += sum of losses > 1e-9, stats[3] += their count (src/trainer/adapt_trainer.cu:237-246)
__global__ void __launch_bounds__(1024) loss_accum_kernel(const float* __restrict__ loss, int n, float* stats) {
    __shared__ float rs[32], rc[32];
    float s = 0.f, c = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float l = loss[i];
        if (l > 1e-9f) { s += l; c += 1.f; }
    }
    s = warp_sum(s); c = warp_sum(c);
    if ((threadIdx.x & 31) == 0) { rs[threadIdx.x >> 5] = s; rc[threadIdx.x >> 5] = c; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float ts = 0.f, tc = 0.f;
        for (int w = 0; w < int(blockDim.x >> 5); w++) { ts += rs[w]; tc += rc[w]; }
        stats[2] += ts; stats[3] += tc;
    }
}

unsigned blocks_for(long n) { return unsigned(std::min<long>(std::max<long>((n + 255) / 256, 1), 148 * 16)); }

void target_dims(const ta_model_config& c, int t, int* in, int* out) {
    const int H = c.hidden, I = c.intermediate, qd = c.q_heads * c.head_dim, kv = c.kv_heads * c.head_dim;
    switch (t) {
        case T_Q: *in = H; *out = qd; break;
        case T_K: case T_V: *in = H; *out = kv; break;
        case T_O: *in = qd; *out = H; break;
        case T_GATE: case T_UP: *in = H; *out = I; break;
        default: *in = I; *out = H; break;
    }
}

#define RC(call) do { if (int _rc = (call)) return _rc; } while (0)

// y = x.W^T (+bias) (+ s.h.B^T) (+residual); keeps h_s in the layer cache for the backward
// h_s of every projection of a fused group in ONE pass over x: the A blocks of the group are contiguous
// in the working array ([n*r][in]) and the result is [BT][n*r], of which each projection owns a slice.
int lora_down_group(ta_trainer* t, int l, int first_tgt, int n, const bf16* x, int BT) {
    LoraRef lr = t->ref(l, first_tgt);
    LoraSlot& sl = t->slot(l, first_tgt);
    GemmSegment g;
    g.A = x; g.lda = sl.in; g.B = lr.A; g.ldb = sl.in; g.K = sl.in;
    GemmOut o;
    o.C = t->cache[l].h[first_tgt]; o.ldc = sl.h_ld; o.alpha = t->scale;
    return seg_gemm(t->ctx, t->stream, BT, n * lr.r, &g, 1, o);
}

int proj_fwd(ta_trainer* t, int l, int tgt, const bf16* x, const bf16* W, const bf16* bias, const bf16* residual,
             bf16* y, int BT, bool h_ready = false) {
    int in, out;
    target_dims(t->mc, tgt, &in, &out);
    GemmSegment seg[2];
    seg[0].A = x; seg[0].lda = in; seg[0].B = W; seg[0].ldb = in; seg[0].K = in;
    int nseg = 1;
    LoraRef lr = t->ref(l, tgt);
    if (lr.on()) {
        bf16* h = t->cache[l].h[tgt];
        if (!h_ready) RC(lora_down(t->ctx, t->stream, x, BT, in, lr, t->scale, h));
        seg[1].A = h; seg[1].lda = t->slot(l, tgt).h_ld; seg[1].B = lr.B; seg[1].ldb = lr.r; seg[1].K = lr.r;
        nseg = 2;
    }
    GemmOut o;
    o.C = y; o.ldc = out; o.bias = bias; o.residual = residual;
    return seg_gemm(t->ctx, t->stream, BT, out, seg, nseg, o);
}

// gate = x.Wg^T (+LoRA), up = x.Wu^T (+LoRA), act = silu(gate)*up as ONE launch: every tile computes 128 gate columns and
// the 128 matching up columns and the epilogue stores all three (proj_fwd x 2 + ops::silu_mul_fwd, qwen2.cu:137-147).
// Needs h_s of both adapters as one [BT][2r] buffer (lora_down_group) when they are on.
int proj_gate_up_swiglu(ta_trainer* t, int l, const bf16* x, int BT) {
    const int H = t->mc.hidden, I = t->mc.intermediate;
    LayerW& w = t->L[l];
    LayerCache& k = t->cache[l];
    GemmSegment seg[2];
    seg[0].A = x; seg[0].lda = H; seg[0].K = H;
    seg[0].B = w.gate_w; seg[0].ldb = H; seg[0].B2 = w.up_w; seg[0].ldb2 = H;
    int nseg = 1;
    LoraRef lg = t->ref(l, T_GATE), lu = t->ref(l, T_UP);
    if (lg.on() && lu.on()) {
        seg[1].A = k.h[T_GATE]; seg[1].lda = t->slot(l, T_GATE).h_ld; seg[1].K = 2 * lg.r; seg[1].k_half = lg.r;
        seg[1].B = lg.B; seg[1].ldb = lg.r; seg[1].B2 = lu.B; seg[1].ldb2 = lu.r;
        nseg = 2;
    }
    GemmOut o;
    o.C = k.gate; o.C2 = k.up; o.C3 = k.act; o.ldc = I; o.epi = 1;
    return seg_gemm(t->ctx, t->stream, BT, I, seg, nseg, o);
}

struct BwdProj { const bf16* dY; const bf16* W; int tgt; };
// Optional fused SwiGLU backward on the product of a backward group (the down projection's dX = d_act): the epilogue
// turns d_act into d_gate / d_up with the forward's gate / up and d_act itself is never stored.
struct SwigluBwd { const bf16* gate = nullptr; const bf16* up = nullptr; bf16* d_gate = nullptr; bf16* d_up = nullptr; };

// dX = sum_i dY_i.W_i + sum_i dh_i.A_i in ONE segmented GEMM; gA_i, gB_i accumulated on the way.
// `fused`: the projections share x and form a fused group (contiguous A / gA blocks, dh slices of one
// [BT][np*r] buffer), so gA of the whole group is one pass over x.
int proj_bwd_group(ta_trainer* t, int l, const bf16* x, const BwdProj* ps, int np, bf16* dX, int BT, bool fused,
                   const SwigluBwd* swiglu = nullptr) {
    GemmSegment seg[kMaxSegments];
    int nseg = 0, in = 0;
    for (int i = 0; i < np; i++) {
        int out;
        target_dims(t->mc, ps[i].tgt, &in, &out);
        GemmSegment& g = seg[nseg++];
        g.A = ps[i].dY; g.lda = out; g.B = ps[i].W; g.ldb = in; g.b_mn = true; g.K = out;
    }
    const int r = t->r_pad;
    for (int i = 0; i < np; i++) {
        LoraRef lr = t->ref(l, ps[i].tgt);
        if (!lr.on()) continue;
        int out;
        target_dims(t->mc, ps[i].tgt, &in, &out);
        const int dh_ld = fused ? np * r : r;
        bf16* dh = fused ? t->dh[0] + i * r : t->dh[i];
        const bf16* h = t->cache[l].h[ps[i].tgt];
        const int h_ld = t->slot(l, ps[i].tgt).h_ld;
        {   // dh_s = bf16(s.dY.B)
            GemmSegment g; g.A = ps[i].dY; g.lda = out; g.B = lr.B; g.ldb = lr.r; g.b_mn = true; g.K = out;
            GemmOut o; o.C = dh; o.ldc = dh_ld; o.alpha = t->scale;
            RC(seg_gemm(t->ctx, t->stream, BT, lr.r, &g, 1, o));
        }
        {   // gB += dY^T.h_s
            GemmSegment g; g.A = ps[i].dY; g.lda = out; g.a_mn = true; g.B = h; g.ldb = h_ld; g.b_mn = true; g.K = BT;
            GemmOut o; o.C = lr.gB; o.ldc = lr.r; o.f32 = true; o.accumulate = true;
            o.split_k = tokens_gemm_splits(t->ctx, out, lr.r, BT); o.split_ws = t->splitk; o.split_ws_bytes = t->splitk_bytes;
            RC(seg_gemm(t->ctx, t->stream, out, lr.r, &g, 1, o));
        }
        if (!fused) {   // gA += dh_s^T.x (tiles [in][r], stored transposed)
            GemmSegment g; g.A = x; g.lda = in; g.a_mn = true; g.B = dh; g.ldb = dh_ld; g.b_mn = true; g.K = BT;
            GemmOut o; o.C = lr.gA; o.ldc = in; o.f32 = true; o.accumulate = true; o.transpose_out = true;
            o.split_k = tokens_gemm_splits(t->ctx, in, lr.r, BT); o.split_ws = t->splitk; o.split_ws_bytes = t->splitk_bytes;
            RC(seg_gemm(t->ctx, t->stream, in, lr.r, &g, 1, o));
        }
        GemmSegment& g = seg[nseg++];
        g.A = dh; g.lda = dh_ld; g.B = lr.A; g.ldb = in; g.b_mn = true; g.K = lr.r;
    }
    if (fused) {   // gA of the whole group: [in][np*r] tiles stored transposed into the contiguous gA blocks
        LoraRef first = t->ref(l, ps[0].tgt);
        GemmSegment g; g.A = x; g.lda = in; g.a_mn = true; g.B = t->dh[0]; g.ldb = np * r; g.b_mn = true; g.K = BT;
        GemmOut o; o.C = first.gA; o.ldc = in; o.f32 = true; o.accumulate = true; o.transpose_out = true;
        o.split_k = tokens_gemm_splits(t->ctx, in, np * r, BT); o.split_ws = t->splitk; o.split_ws_bytes = t->splitk_bytes;
        RC(seg_gemm(t->ctx, t->stream, in, np * r, &g, 1, o));
    }
    GemmOut o;
    o.C = dX; o.ldc = in;
    if (swiglu) { o.epi = 2; o.C = swiglu->d_gate; o.C2 = swiglu->d_up; o.gate_in = swiglu->gate; o.up_in = swiglu->up; }
    return seg_gemm(t->ctx, t->stream, BT, in, seg, nseg, o);
}

// forward + loss + backward for one micro-batch already resident in t->tok / t->tgt
// `exchange`: this is the last micro-batch of the optimiser step and a communicator is attached - each layer's
// gradient slice is all-reduced on the communicator's stream as soon as that layer's backward has been issued.
int run_micro(ta_trainer* t, int Bm, int T, float inv_count, bool exchange) {
    const ta_model_config& c = t->mc;
    ta_ctx* ctx = t->ctx;
    void* s = t->stream;
    const int BT = Bm * T, H = c.hidden, I = c.intermediate, qd = c.q_heads * c.head_dim, kv = c.kv_heads * c.head_dim;
    const int Lyr = c.layers;
    // SwiGLU folded into the GEMM epilogues (no act / d_act round trips) whenever the 256-row tile kernels apply
    const bool swiglu_fused = t->fuse_swiglu < 0 ? seg_gemm_swiglu_pays(ctx, BT) : (t->fuse_swiglu != 0 && seg_gemm_supports_swiglu(ctx, BT));

    // ── forward ────────────────────────────────────────────────────────────
    RC(ta_embed_fwd(ctx, t->embed, t->tok, t->cache[0].r_in, BT, H, s));
    for (int l = 0; l < Lyr; l++) {
        LayerW& w = t->L[l];
        LayerCache& k = t->cache[l];
        bf16* r_next = (l + 1 < Lyr) ? t->cache[l + 1].r_in : t->r_final;
        RC(ta_rms_norm_fwd(ctx, k.r_in, w.input_norm, k.x_normed, k.in_rms, BT, H, c.rms_eps, s));
        if (t->fuse_qkv) RC(lora_down_group(t, l, T_Q, 3, k.x_normed, BT));
        RC(proj_fwd(t, l, T_Q, k.x_normed, w.q_w, w.q_b, nullptr, k.Q, BT, t->fuse_qkv));
        RC(proj_fwd(t, l, T_K, k.x_normed, w.k_w, w.k_b, nullptr, k.K, BT, t->fuse_qkv));
        RC(proj_fwd(t, l, T_V, k.x_normed, w.v_w, w.v_b, nullptr, k.V, BT, t->fuse_qkv));
        RC(ta_rope(ctx, k.Q, c.q_heads, k.K, c.kv_heads, Bm, T, c.head_dim, c.rope_theta, 0, s));
        RC(ta_flash_attn_fwd(ctx, k.Q, k.K, k.V, k.attn_out, k.lse, Bm, T, c.q_heads, c.kv_heads, c.head_dim, s));
        RC(proj_fwd(t, l, T_O, k.attn_out, w.o_w, nullptr, k.r_in, k.r_mid, BT));          // + residual
        RC(ta_rms_norm_fwd(ctx, k.r_mid, w.post_norm, k.x_normed2, k.post_rms, BT, H, c.rms_eps, s));
        if (t->fuse_gu) RC(lora_down_group(t, l, T_GATE, 2, k.x_normed2, BT));
        if (swiglu_fused && (t->fuse_gu || (!t->ref(l, T_GATE).on() && !t->ref(l, T_UP).on()))) {
            RC(proj_gate_up_swiglu(t, l, k.x_normed2, BT));
        } else {
            RC(proj_fwd(t, l, T_GATE, k.x_normed2, w.gate_w, nullptr, nullptr, k.gate, BT, t->fuse_gu));
            RC(proj_fwd(t, l, T_UP, k.x_normed2, w.up_w, nullptr, nullptr, k.up, BT, t->fuse_gu));
            RC(ta_silu_mul_fwd(ctx, k.gate, k.up, k.act, long(BT) * I, s));
        }
        RC(proj_fwd(t, l, T_DOWN, k.act, w.down_w, nullptr, k.r_mid, r_next, BT));         // + residual
    }
    RC(ta_rms_norm_fwd(ctx, t->r_final, t->final_norm, t->x_final_normed, t->final_rms, BT, H, c.rms_eps, s));

    // ── lm head + cross-entropy + head backward, in row chunks so [BT,V] never exists at once ──
    const bf16* lm = c.tie_embeddings ? t->embed : t->lm_head;
    RC(ta_lmhead_ce_fwd_bwd(ctx, t->x_final_normed, lm, t->tgt, t->loss, t->d_xn, BT, H, c.vocab, inv_count, t->logits,
                            t->logit_rows, s));
    loss_accum_kernel<<<1, 1024, 0, t->stream>>>(t->loss, BT, t->stats);
    TA_LAUNCH_CHECK(ctx, "loss_accum_kernel");
    // grad = rms_norm_bwd(dres, x_final, final_norm)                         (qwen2.cu:203-213)
    RC(ta_rms_norm_bwd(ctx, t->d_xn, t->r_final, t->final_norm, t->final_rms, t->g_res, nullptr, BT, H, s));

    // ── backward ───────────────────────────────────────────────────────────
    for (int l = Lyr - 1; l >= 0; l--) {
        LayerW& w = t->L[l];
        LayerCache& k = t->cache[l];
        {   // FFN: dact = grad.Wd (+LoRA down), then dgate / dup                (qwen2.cu:221-230)
            BwdProj p{t->g_res, w.down_w, T_DOWN};
            if (swiglu_fused) {
                SwigluBwd sw; sw.gate = k.gate; sw.up = k.up; sw.d_gate = t->d_gate; sw.d_up = t->d_up;
                RC(proj_bwd_group(t, l, k.act, &p, 1, nullptr, BT, false, &sw));
            } else {
                RC(proj_bwd_group(t, l, k.act, &p, 1, t->d_act, BT, false));
                RC(ta_silu_mul_bwd(ctx, t->d_act, k.gate, k.up, t->d_gate, t->d_up, long(BT) * I, s));
            }
        }
        {   // dx_normed2 = dgate.Wg + dup.Wu (+LoRA)                           (:232-234)
            BwdProj p[2] = {{t->d_gate, w.gate_w, T_GATE}, {t->d_up, w.up_w, T_UP}};
            RC(proj_bwd_group(t, l, k.x_normed2, p, 2, t->d_xn, BT, t->fuse_gu));
        }
        // grad += rms_norm_bwd(dx_normed2, pre_ffn_res)                       (:238-246)
        RC(ta_rms_norm_bwd(ctx, t->d_xn, k.r_mid, w.post_norm, k.post_rms, t->g_res, t->g_res, BT, H, s));
        {   // dx_attn_out = grad.Wo (+LoRA o)                                 (:253-264)
            BwdProj p{t->g_res, w.o_w, T_O};
            RC(proj_bwd_group(t, l, k.attn_out, &p, 1, t->d_attn, BT, false));
        }
        RC(ta_flash_attn_bwd(ctx, t->d_attn, k.Q, k.K, k.V, k.attn_out, k.lse, t->dQ, t->dK, t->dV, t->delta, Bm, T,
                             c.q_heads, c.kv_heads, c.head_dim, s));
        RC(ta_rope(ctx, t->dQ, c.q_heads, t->dK, c.kv_heads, Bm, T, c.head_dim, c.rope_theta, 1, s));
        {   // dx_normed = dQ.Wq + dK.Wk + dV.Wv (+LoRA q,k,v)                  (:282-292)
            BwdProj p[3] = {{t->dQ, w.q_w, T_Q}, {t->dK, w.k_w, T_K}, {t->dV, w.v_w, T_V}};
            RC(proj_bwd_group(t, l, k.x_normed, p, 3, t->d_xn, BT, t->fuse_qkv));
        }
        // centroid side-channel: hidden = x_normed, signal = dx_normed        (adapt_trainer.cu:210-232)
        if (t->ac.centroid_modes & 1)
            RC(ta_centroid_accumulate(ctx, TA_CENTROID_INTENDED, k.x_normed, t->d_xn, BT, H, t->cen_acc, t->cen_w, s));
        if (t->ac.centroid_modes & 2)
            RC(ta_centroid_accumulate(ctx, TA_CENTROID_ASBUILT, k.x_normed, t->d_xn, BT, H, t->cen_acc_ab, t->cen_w_ab, s));
        if (t->ac.centroid_modes & 4)   // per-layer bank: the documented sum kept separately for every layer
            RC(ta_centroid_accumulate(ctx, TA_CENTROID_INTENDED, k.x_normed, t->d_xn, BT, H, t->cen_bank + size_t(l) * H,
                                      t->cen_bank_w + l, s));
        // grad += rms_norm_bwd(dx_normed, pre_attn_res)                       (:298-304)
        if (l > 0)
            RC(ta_rms_norm_bwd(ctx, t->d_xn, k.r_in, w.input_norm, k.in_rms, t->g_res, t->g_res, BT, H, s));
        if (exchange) RC(comm_reduce_slice(t, t->layer_begin[size_t(l)], t->layer_begin[size_t(l) + 1]));
    }
    if (exchange) RC(comm_finish_step(t));
    (void)qd; (void)kv;
    return TA_OK;
}

size_t bytes_bf16(long n) { return size_t(n) * 2; }

}  // namespace
}  // namespace ta

using namespace ta;

extern "C" {

int ta_trainer_create(ta_ctx* ctx, const ta_model_config* mc, const ta_adapter_config* ac, int micro_batch, int seq_len,
                      void* stream, ta_trainer** out) {
    if (!ctx || !mc || !ac || !out || micro_batch <= 0 || seq_len <= 0)
        return fail(ctx, TA_ERR_INVALID, "trainer_create: null argument or bad size");
    *out = nullptr;
    const ta_model_config& c = *mc;
    if (c.vocab <= 0 || c.hidden <= 0 || c.layers <= 0 || c.q_heads <= 0 || c.kv_heads <= 0 || c.intermediate <= 0 ||
        c.q_heads % c.kv_heads != 0)
        return fail(ctx, TA_ERR_INVALID, "trainer_create: bad model config");
    if (c.head_dim != 64 && c.head_dim != 128) return fail(ctx, TA_ERR_UNSUPPORTED, "trainer_create: head_dim 64 or 128");
    if (c.hidden % 8 || c.intermediate % 8 || c.vocab % 8) return fail(ctx, TA_ERR_UNSUPPORTED, "trainer_create: dims % 8");
    if (ac->rank <= 0 || ac->rank > 256) return fail(ctx, TA_ERR_INVALID, "trainer_create: rank must be in 1..256");

    ta_trainer* t = new ta_trainer();
    t->ctx = ctx; t->stream = static_cast<cudaStream_t>(stream); t->mc = c; t->ac = *ac;
    t->r_pad = (ac->rank + 15) / 16 * 16;
    t->scale = ac->alpha / float(ac->rank);
    t->micro_B = micro_batch; t->T = seq_len;
    const long H = c.hidden, I = c.intermediate, V = c.vocab, qd = long(c.q_heads) * c.head_dim,
               kv = long(c.kv_heads) * c.head_dim, BT = long(micro_batch) * seq_len;
    const int Lyr = c.layers, r = t->r_pad;

    auto fail_free = [&](int code, const char* msg) { ta_trainer_destroy(t); return fail(ctx, code, msg); };

    // pass 0 measures, pass 1 assigns (the arenas hand out null pointers until they have a base)
    for (int pass = 0; pass < 2; pass++) {
        DeviceArena& W = t->weights; DeviceArena& Lo = t->lora; DeviceArena& A = t->acts;
        W.used = Lo.used = A.used = 0;
        // frozen base
        t->embed = static_cast<bf16*>(W.take(bytes_bf16(V * H)));
        t->final_norm = static_cast<bf16*>(W.take(bytes_bf16(H)));
        t->lm_head = c.tie_embeddings ? nullptr : static_cast<bf16*>(W.take(bytes_bf16(V * H)));
        t->L.resize(Lyr);
        for (int l = 0; l < Lyr; l++) {
            LayerW& w = t->L[l];
            w.input_norm = static_cast<bf16*>(W.take(bytes_bf16(H)));
            w.post_norm = static_cast<bf16*>(W.take(bytes_bf16(H)));
            w.q_w = static_cast<bf16*>(W.take(bytes_bf16(qd * H)));
            w.k_w = static_cast<bf16*>(W.take(bytes_bf16(kv * H)));
            w.v_w = static_cast<bf16*>(W.take(bytes_bf16(kv * H)));
            w.o_w = static_cast<bf16*>(W.take(bytes_bf16(H * qd)));
            w.q_b = static_cast<bf16*>(W.take(bytes_bf16(qd)));
            w.k_b = static_cast<bf16*>(W.take(bytes_bf16(kv)));
            w.v_b = static_cast<bf16*>(W.take(bytes_bf16(kv)));
            w.gate_w = static_cast<bf16*>(W.take(bytes_bf16(I * H)));
            w.up_w = static_cast<bf16*>(W.take(bytes_bf16(I * H)));
            w.down_w = static_cast<bf16*>(W.take(bytes_bf16(H * I)));
        }
        // LoRA slots: offsets in elements, each block padded to 128 elements.  Projections that read the
        // same input (q/k/v, gate/up) get their A blocks back to back - and, as all five arrays share the
        // offsets, their gA blocks too - so one GEMM serves the whole group.
        t->slots.assign(size_t(Lyr) * T_COUNT, LoraSlot());
        auto on = [&](int tg) { return (ac->targets & (1 << tg)) != 0; };
        t->fuse_qkv = on(T_Q) && on(T_K) && on(T_V);
        t->fuse_gu = on(T_GATE) && on(T_UP);
        long off = 0;
        size_t sk_need = 0;
        t->layer_begin.assign(size_t(Lyr) + 1, 0);
        static const int kGroups[4][3] = {{T_Q, T_K, T_V}, {T_O, -1, -1}, {T_GATE, T_UP, -1}, {T_DOWN, -1, -1}};
        for (int l = 0; l < Lyr; l++) {
            t->layer_begin[size_t(l)] = off;
            for (const auto& grp : kGroups) {
                int members[3], nm = 0;
                for (int tg : grp) if (tg >= 0 && on(tg)) members[nm++] = tg;
                const bool fused = (grp[0] == T_Q && t->fuse_qkv) || (grp[0] == T_GATE && t->fuse_gu);
                for (int i = 0; i < nm; i++) {   // all A blocks of the group first ...
                    LoraSlot& sl = t->slot(l, members[i]);
                    sl.on = true;
                    target_dims(c, members[i], &sl.in, &sl.out);
                    sl.h_ld = fused ? nm * r : r;
                    sl.offA = off; off += (long(r) * sl.in + 127) / 128 * 128;
                }
                for (int i = 0; i < nm; i++) {   // ... then the B blocks
                    LoraSlot& sl = t->slot(l, members[i]);
                    sl.offB = off; off += (long(sl.out) * r + 127) / 128 * 128;
                    sk_need = std::max({sk_need, tokens_gemm_ws_bytes_max(ctx, sl.out, r),
                                        tokens_gemm_ws_bytes_max(ctx, sl.in, fused ? nm * r : r)});
                }
            }
        }
        t->layer_begin[size_t(Lyr)] = off;
        t->lora_n = off;
        t->master = static_cast<float*>(Lo.take(size_t(off) * 4));
        t->m = static_cast<float*>(Lo.take(size_t(off) * 4));
        t->v = static_cast<float*>(Lo.take(size_t(off) * 4));
        t->grad = static_cast<float*>(Lo.take(size_t(off) * 4));
        t->working = static_cast<bf16*>(Lo.take(size_t(off) * 2));
        t->cen_acc = static_cast<float*>(Lo.take(size_t(H) * 4));
        t->cen_acc_ab = static_cast<float*>(Lo.take(size_t(H) * 4));
        t->cen_bank = static_cast<float*>(Lo.take(size_t(Lyr) * H * 4));
        t->cen_bank_w = static_cast<float*>(Lo.take(size_t(Lyr) * 4));
        t->cen_w = static_cast<float*>(Lo.take(256));
        t->cen_w_ab = t->cen_w + 1;
        t->stats = t->cen_w + 8;
        // activations
        t->cache.resize(Lyr);
        for (int l = 0; l < Lyr; l++) {
            LayerCache& k = t->cache[l];
            k.r_in = static_cast<bf16*>(A.take(bytes_bf16(BT * H)));
            k.x_normed = static_cast<bf16*>(A.take(bytes_bf16(BT * H)));
            k.Q = static_cast<bf16*>(A.take(bytes_bf16(BT * qd)));
            k.K = static_cast<bf16*>(A.take(bytes_bf16(BT * kv)));
            k.V = static_cast<bf16*>(A.take(bytes_bf16(BT * kv)));
            k.attn_out = static_cast<bf16*>(A.take(bytes_bf16(BT * qd)));
            k.r_mid = static_cast<bf16*>(A.take(bytes_bf16(BT * H)));
            k.x_normed2 = static_cast<bf16*>(A.take(bytes_bf16(BT * H)));
            k.gate = static_cast<bf16*>(A.take(bytes_bf16(BT * I)));
            k.up = static_cast<bf16*>(A.take(bytes_bf16(BT * I)));
            k.act = static_cast<bf16*>(A.take(bytes_bf16(BT * I)));
            k.in_rms = static_cast<float*>(A.take(size_t(BT) * 4));
            k.post_rms = static_cast<float*>(A.take(size_t(BT) * 4));
            k.lse = static_cast<float*>(A.take(size_t(BT) * c.q_heads * 4));
            for (int tg = 0; tg < T_COUNT; tg++) k.h[tg] = nullptr;
            if (t->fuse_qkv) {
                bf16* hb = static_cast<bf16*>(A.take(bytes_bf16(BT * 3 * r)));
                k.h[T_Q] = hb; k.h[T_K] = hb ? hb + r : nullptr; k.h[T_V] = hb ? hb + 2 * r : nullptr;
            }
            if (t->fuse_gu) {
                bf16* hb = static_cast<bf16*>(A.take(bytes_bf16(BT * 2 * r)));
                k.h[T_GATE] = hb; k.h[T_UP] = hb ? hb + r : nullptr;
            }
            for (int tg = 0; tg < T_COUNT; tg++)
                if (t->slot(l, tg).on && !k.h[tg] && !((tg <= T_V && t->fuse_qkv) || ((tg == T_GATE || tg == T_UP) && t->fuse_gu)))
                    k.h[tg] = static_cast<bf16*>(A.take(bytes_bf16(BT * r)));
        }
        t->r_final = static_cast<bf16*>(A.take(bytes_bf16(BT * H)));
        t->x_final_normed = static_cast<bf16*>(A.take(bytes_bf16(BT * H)));
        t->final_rms = static_cast<float*>(A.take(size_t(BT) * 4));
        long lr_rows = std::max<long>(128, std::min<long>(BT, (long(2500000000ll) / (V * 2)) / 128 * 128));
        t->logit_rows = int(std::min<long>(lr_rows, (BT + 127) / 128 * 128));
        t->logits = static_cast<bf16*>(A.take(bytes_bf16(long(t->logit_rows) * V)));
        t->g_res = static_cast<bf16*>(A.take(bytes_bf16(BT * H)));
        t->d_act = static_cast<bf16*>(A.take(bytes_bf16(BT * I)));
        t->d_gate = static_cast<bf16*>(A.take(bytes_bf16(BT * I)));
        t->d_up = static_cast<bf16*>(A.take(bytes_bf16(BT * I)));
        t->d_xn = static_cast<bf16*>(A.take(bytes_bf16(BT * H)));
        t->d_attn = static_cast<bf16*>(A.take(bytes_bf16(BT * qd)));
        t->dQ = static_cast<bf16*>(A.take(bytes_bf16(BT * qd)));
        t->dK = static_cast<bf16*>(A.take(bytes_bf16(BT * kv)));
        t->dV = static_cast<bf16*>(A.take(bytes_bf16(BT * kv)));
        {   // one [BT][3r] block: separate projections use r-wide thirds, a fused group uses slices of it
            bf16* db = static_cast<bf16*>(A.take(bytes_bf16(BT * 3 * r)));
            for (int i = 0; i < 3; i++) t->dh[i] = db ? db + long(i) * BT * r : nullptr;
        }
        t->delta = static_cast<float*>(A.take(size_t(BT) * c.q_heads * 4));
        t->splitk_bytes = sk_need + 256;
        t->splitk = static_cast<float*>(A.take(t->splitk_bytes));
        t->loss = static_cast<float*>(A.take(size_t(BT) * 4));
        t->tok = static_cast<int*>(A.take(size_t(BT) * 4));
        t->tgt = static_cast<int*>(A.take(size_t(BT) * 4));
        if (pass == 0) {
            for (DeviceArena* a : {&W, &Lo, &A}) {
                a->size = a->used + 256;
                void* p = nullptr;
                if (cudaMalloc(&p, a->size) != cudaSuccess) {
                    cudaGetLastError();
                    return fail_free(TA_ERR_NOMEM, "trainer_create: cudaMalloc failed (model + activations do not fit)");
                }
                a->base = static_cast<char*>(p);
            }
        }
    }
    if (cudaMallocHost(reinterpret_cast<void**>(&t->h_stats), 64) != cudaSuccess)
        return fail_free(TA_ERR_NOMEM, "trainer_create: pinned host allocation failed");
    // LoRA state: zeros everywhere, then the reference's Kaiming values into each logical A block
    cudaStream_t s = t->stream;
    cudaMemsetAsync(t->lora.base, 0, t->lora.size, s);
    for (int l = 0; l < Lyr; l++)
        for (int tg = 0; tg < T_COUNT; tg++) {
            LoraSlot& sl = t->slot(l, tg);
            if (!sl.on) continue;
            const int n = ac->rank * sl.in;
            kaiming_kernel<<<(n + 255) / 256, 256, 0, s>>>(t->master + sl.offA, sl.in, ac->rank, 0x1234u);
        }
    if (cudaGetLastError() != cudaSuccess) return fail_free(TA_ERR_CUDA, "trainer_create: init kernels failed");
    if (int rc = ta_trainer_sync_working(t)) { ta_trainer_destroy(t); return rc; }
    *out = t;
    return TA_OK;
}

int ta_trainer_destroy(ta_trainer* t) {
    if (!t) return TA_OK;
    cudaDeviceSynchronize();
    for (DeviceArena* a : {&t->weights, &t->lora, &t->acts})
        if (a->base) cudaFree(a->base);
    if (t->h_stats) cudaFreeHost(t->h_stats);
    // tensor maps of freed memory must not be served again
    if (t->ctx) t->ctx->tmaps.clear();
    delete t;
    return TA_OK;
}

int ta_trainer_init_random(ta_trainer* t, unsigned long long seed, float stdv) {
    if (!t) return TA_ERR_INVALID;
    const ta_model_config& c = t->mc;
    const long H = c.hidden, I = c.intermediate, V = c.vocab, qd = long(c.q_heads) * c.head_dim,
               kv = long(c.kv_heads) * c.head_dim;
    cudaStream_t s = t->stream;
    unsigned long long k = seed * 1000003ull;
    auto nrm = [&](bf16* p, long n) { fill_normal_kernel<<<blocks_for(n), 256, 0, s>>>(p, n, stdv, ++k); };
    auto one = [&](bf16* p, long n) { fill_const_kernel<<<blocks_for(n), 256, 0, s>>>(p, n, 1.f); };
    nrm(t->embed, V * H); one(t->final_norm, H);
    if (t->lm_head) nrm(t->lm_head, V * H);
    for (auto& w : t->L) {
        one(w.input_norm, H); one(w.post_norm, H);
        nrm(w.q_w, qd * H); nrm(w.k_w, kv * H); nrm(w.v_w, kv * H); nrm(w.o_w, H * qd);
        nrm(w.q_b, qd); nrm(w.k_b, kv); nrm(w.v_b, kv);
        nrm(w.gate_w, I * H); nrm(w.up_w, I * H); nrm(w.down_w, H * I);
    }
    TA_LAUNCH_CHECK(t->ctx, "fill kernels");
    return TA_OK;
}

int ta_trainer_tensor(ta_trainer* t, const char* name, void** dev_ptr, long* rows, long* cols, long* pitch, int* dtype) {
    if (!t || !name || !dev_ptr) return TA_ERR_INVALID;
    const ta_model_config& c = t->mc;
    const long H = c.hidden, I = c.intermediate, V = c.vocab, qd = long(c.q_heads) * c.head_dim,
               kv = long(c.kv_heads) * c.head_dim, BT = long(t->micro_B) * t->T;
    void* p = nullptr; long r = 1, cc = 1, pt = -1; int dt = 1;
    std::string n(name);
    auto set = [&](void* q, long rr, long c2, int d, long pitch_ = -1) { p = q; r = rr; cc = c2; dt = d; pt = pitch_ < 0 ? c2 : pitch_; };
    int l = -1; char rest[64] = {0};
    if (n == "embed") set(t->embed, V, H, 1);
    else if (n == "final_norm") set(t->final_norm, 1, H, 1);
    else if (n == "lm_head") set(t->lm_head, V, H, 1);
    else if (n == "lora.master") set(t->master, 1, t->lora_n, 0);
    else if (n == "lora.grad") set(t->grad, 1, t->lora_n, 0);
    else if (n == "lora.m") set(t->m, 1, t->lora_n, 0);
    else if (n == "lora.v") set(t->v, 1, t->lora_n, 0);
    else if (n == "lora.working") set(t->working, 1, t->lora_n, 1);
    else if (n == "step.stats") set(t->stats, 1, 4, 0);   // [grad norm, clip scale, loss sum, loss count]
    else if (n == "centroid.acc") set(t->cen_acc, 1, H, 0);
    else if (n == "centroid.weight") set(t->cen_w, 1, 1, 0);
    else if (n == "centroid_asbuilt.acc") set(t->cen_acc_ab, 1, H, 0);
    else if (n == "centroid_asbuilt.weight") set(t->cen_w_ab, 1, 1, 0);
    else if (n == "centroid_bank.acc") set(t->cen_bank, c.layers, H, 0);
    else if (n == "centroid_bank.weight") set(t->cen_bank_w, 1, c.layers, 0);
    else if (n == "cache.dx_attn_in") set(t->d_xn, BT, H, 1);
    else if (n == "cache.loss") set(t->loss, 1, BT, 0);
    else if (n == "cache.dQ") set(t->dQ, BT, qd, 1);
    else if (n == "cache.dK") set(t->dK, BT, kv, 1);
    else if (n == "cache.dV") set(t->dV, BT, kv, 1);
    else if (n == "cache.d_attn_out") set(t->d_attn, BT, qd, 1);
    else if (std::sscanf(name, "l%d.%63s", &l, rest) == 2 && l >= 0 && l < c.layers) {
        std::string f(rest);
        LayerW& w = t->L[l];
        LayerCache& k = t->cache[l];
        if (f == "input_norm") set(w.input_norm, 1, H, 1);
        else if (f == "post_norm") set(w.post_norm, 1, H, 1);
        else if (f == "q_w") set(w.q_w, qd, H, 1);
        else if (f == "k_w") set(w.k_w, kv, H, 1);
        else if (f == "v_w") set(w.v_w, kv, H, 1);
        else if (f == "o_w") set(w.o_w, H, qd, 1);
        else if (f == "q_b") set(w.q_b, 1, qd, 1);
        else if (f == "k_b") set(w.k_b, 1, kv, 1);
        else if (f == "v_b") set(w.v_b, 1, kv, 1);
        else if (f == "gate_w") set(w.gate_w, I, H, 1);
        else if (f == "up_w") set(w.up_w, I, H, 1);
        else if (f == "down_w") set(w.down_w, H, I, 1);
        else if (f == "cache.x_normed") set(k.x_normed, BT, H, 1);
        else if (f == "cache.Q") set(k.Q, BT, qd, 1);
        else if (f == "cache.K") set(k.K, BT, kv, 1);
        else if (f == "cache.V") set(k.V, BT, kv, 1);
        else if (f == "cache.attn_out") set(k.attn_out, BT, qd, 1);
        else if (f == "cache.r_in") set(k.r_in, BT, H, 1);
        else if (f == "cache.r_mid") set(k.r_mid, BT, H, 1);
        else if (f.rfind("lora.", 0) == 0) {
            const size_t dot = f.find('.', 5);
            if (dot == std::string::npos) return fail(t->ctx, TA_ERR_INVALID, "trainer_tensor: bad lora name");
            const std::string tn = f.substr(5, dot - 5), which = f.substr(dot + 1);
            int tg = -1;
            for (int i = 0; i < T_COUNT; i++) if (tn == kTargetNames[i]) tg = i;
            if (tg < 0 || !t->slot(l, tg).on) return fail(t->ctx, TA_ERR_INVALID, "trainer_tensor: no such adapter");
            LoraSlot& sl = t->slot(l, tg);
            const bool isA = which == "A" || which == "gA" || which == "mA" || which == "vA" || which == "A_bf16";
            const long off = isA ? sl.offA : sl.offB;
            const long rr = isA ? t->ac.rank : sl.out, c2 = isA ? sl.in : t->ac.rank, pp = isA ? sl.in : t->r_pad;
            if (which == "A" || which == "B") set(t->master + off, rr, c2, 0, pp);
            else if (which == "gA" || which == "gB") set(t->grad + off, rr, c2, 0, pp);
            else if (which == "mA" || which == "mB") set(t->m + off, rr, c2, 0, pp);
            else if (which == "vA" || which == "vB") set(t->v + off, rr, c2, 0, pp);
            else if (which == "A_bf16" || which == "B_bf16") set(t->working + off, rr, c2, 1, pp);
            else return fail(t->ctx, TA_ERR_INVALID, "trainer_tensor: bad lora field");
        } else return fail(t->ctx, TA_ERR_INVALID, std::string("trainer_tensor: unknown name ") + name);
    } else return fail(t->ctx, TA_ERR_INVALID, std::string("trainer_tensor: unknown name ") + name);
    if (!p) return fail(t->ctx, TA_ERR_INVALID, std::string("trainer_tensor: tensor not present: ") + name);
    *dev_ptr = p;
    if (rows) *rows = r;
    if (cols) *cols = cc;
    if (pitch) *pitch = pt;
    if (dtype) *dtype = dt;
    return TA_OK;
}

int ta_trainer_set_option(ta_trainer* t, const char* name, int value) {
    if (!t || !name) return TA_ERR_INVALID;
    if (!std::strcmp(name, "fuse_swiglu")) { t->fuse_swiglu = value < 0 ? -1 : (value != 0); return TA_OK; }
    return fail(t->ctx, TA_ERR_INVALID, std::string("trainer_set_option: unknown option ") + name);
}

int ta_trainer_sync_working(ta_trainer* t) {
    if (!t) return TA_ERR_INVALID;
    return ta_cast_f32_to_bf16(t->ctx, t->master, t->working, t->lora_n, t->stream);
}

int ta_trainer_zero_grad(ta_trainer* t) {
    if (!t) return TA_ERR_INVALID;
    TA_CUDA(t->ctx, cudaMemsetAsync(t->grad, 0, size_t(t->lora_n) * 4, t->stream));
    TA_CUDA(t->ctx, cudaMemsetAsync(t->stats, 0, 4 * sizeof(float), t->stream));
    return TA_OK;
}

int ta_trainer_forward_backward(ta_trainer* t, const int* tokens, const int* targets, int B, int T, long global_tokens,
                                int host_inputs) {
    if (!t || !tokens || !targets || B <= 0 || T <= 0) return fail(t ? t->ctx : nullptr, TA_ERR_INVALID, "forward_backward: bad argument");
    if (T != t->T) return fail(t->ctx, TA_ERR_INVALID, "forward_backward: T differs from the trainer's seq_len");
    // Tokens are counted once per optimiser step: a caller that names the step's global token count (a
    // data-parallel rank, or several accumulating calls) has exactly that many consumed by the step, as
    // AdaptTrainer counts batch_size * seq_len per step (src/trainer/adapt_trainer.cu:255-256).
    if (global_tokens > 0) t->pending_tokens = global_tokens;
    else { global_tokens = long(B) * T; t->pending_tokens += global_tokens; }
    const float inv = 1.f / float(global_tokens);
    const cudaMemcpyKind kind = host_inputs ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice;
    for (int b0 = 0; b0 < B; b0 += t->micro_B) {
        const int Bm = std::min(t->micro_B, B - b0);
        const size_t bytes = size_t(Bm) * T * sizeof(int);
        TA_CUDA(t->ctx, cudaMemcpyAsync(t->tok, tokens + size_t(b0) * T, bytes, kind, t->stream));
        TA_CUDA(t->ctx, cudaMemcpyAsync(t->tgt, targets + size_t(b0) * T, bytes, kind, t->stream));
        if (int rc = run_micro(t, Bm, T, inv, t->comm != nullptr && b0 + t->micro_B >= B)) return rc;
    }
    return TA_OK;
}

int ta_trainer_optimizer_step(ta_trainer* t, float lr, long total_steps, ta_step_metrics* out) {
    if (!t) return TA_ERR_INVALID;
    const ta_adapter_config& a = t->ac;
    if (lr < 0.f) lr = ta_cosine_lr(a.lr, a.warmup_steps, total_steps, t->step_count, 0.1f);
    const int step = int(t->step_count) + 1;
    if (int rc = ta_gradnorm_clip_adamw(t->ctx, t->master, t->working, t->m, t->v, t->grad, t->lora_n, lr, a.beta1, a.beta2,
                                        a.eps, a.weight_decay, step, a.grad_clip, t->stats, 1, t->stream))
        return rc;
    TA_CUDA(t->ctx, cudaMemcpyAsync(t->h_stats, t->stats, 4 * sizeof(float), cudaMemcpyDeviceToHost, t->stream));
    TA_CUDA(t->ctx, cudaStreamSynchronize(t->stream));
    t->step_count++;
    t->tokens_seen += t->pending_tokens;
    t->pending_tokens = 0;
    if (out) {
        out->step = t->step_count;
        out->tokens_consumed = t->tokens_seen;
        out->loss = t->h_stats[3] > 0.f ? t->h_stats[2] / t->h_stats[3] : 0.f;
        out->learning_rate = lr;
        out->grad_norm_raw = t->h_stats[0];
        out->grad_norm = a.grad_clip > 0.f ? std::min(t->h_stats[0], a.grad_clip) : t->h_stats[0];
    }
    int st = 0;
    return ta_device_status(t->ctx, &st);
}

int ta_trainer_step(ta_trainer* t, const int* tokens, const int* targets, int B, int T, float lr, long total_steps,
                    int host_inputs, ta_step_metrics* out) {
    if (int rc = ta_trainer_zero_grad(t)) return rc;
    if (int rc = ta_trainer_forward_backward(t, tokens, targets, B, T, long(B) * T, host_inputs)) return rc;
    return ta_trainer_optimizer_step(t, lr, total_steps, out);
}

float ta_cosine_lr(float base_lr, long warmup_steps, long total_steps, long step, float floor_frac) {
    if (step < warmup_steps) return base_lr * float(step + 1) / float(warmup_steps);
    float progress = float(step - warmup_steps) / float(total_steps - warmup_steps);
    progress = std::min(progress, 1.f);
    const float cos_val = 0.5f * (1.f + std::cos(3.14159265358979323846f * progress));
    const float floor_lr = base_lr * floor_frac;
    return floor_lr + (base_lr - floor_lr) * cos_val;
}

void ta_mask_targets(const int* ids, int* tgt, int B, int T) {
    constexpr int IM_START = 151644, ASSISTANT = 77091, IM_END = 151645;
    for (int b = 0; b < B; b++) {
        bool inside = false;
        for (int i = 0; i < T; i++) {
            const int idx = b * T + i, tok = ids[idx];
            if (tok == IM_START) inside = (i + 1 < T && ids[idx + 1] == ASSISTANT);
            bool mask = !inside;
            if (tok == IM_START || tok == ASSISTANT) mask = true;
            if (tok == IM_END) { inside = false; mask = false; }
            if (mask) tgt[idx] = -1;
        }
    }
}

void ta_kaiming_init_host(float* out, int in_dim, int rank, unsigned seed) {
    for (int i = 0; i < in_dim * rank; i++) out[i] = kaiming_value(unsigned(i), in_dim, seed);
}

int ta_memcpy_h2d(void* dst, const void* src, size_t bytes) {
    return cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice) == cudaSuccess ? TA_OK : TA_ERR_CUDA;
}
int ta_memcpy_d2h(void* dst, const void* src, size_t bytes) {
    return cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost) == cudaSuccess ? TA_OK : TA_ERR_CUDA;
}

}  // extern "C"
