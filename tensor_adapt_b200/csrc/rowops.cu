// HBM-bound kernels of the training step: RMSNorm, RoPE, SwiGLU, embedding gather, residual / bias
// adds, casts and cross-entropy.  All use 16-byte vector accesses, FP32 arithmetic inside, and
// warp-shuffle reductions; none allocates memory.
#include <algorithm>
#include <cfloat>

#include "ctx.h"
#include "ptx.cuh"

namespace ta {
namespace {

constexpr int kMaxVec = 8;   // per-thread 16-byte vectors held in registers by the row kernels

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 t = unpack_bf16x2(w[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 u;
    u.x = pack_bf16x2(f[0], f[1]);
    u.y = pack_bf16x2(f[2], f[3]);
    u.z = pack_bf16x2(f[4], f[5]);
    u.w = pack_bf16x2(f[6], f[7]);
    return u;
}

// Block-wide sum of one float per thread; every thread gets the result. `red` has >= 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();   // protect `red` from the previous use
    if (lane == 0) red[w] = v;
    __syncthreads();
    if (w == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// ── RMSNorm ─────────────────────────────────────────────────────────────────
// One CTA walks rows grid-stride; a row of D bf16 is read ONCE into registers (<= kMaxVec 16-byte
// vectors per thread), reduced, scaled and written.  Algorithmic traffic: 2*D*2 bytes + 4 per row.

template <int NT>
__global__ void __launch_bounds__(NT) rms_norm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ w,
                                                          __nv_bfloat16* __restrict__ out, float* __restrict__ rms_out,
                                                          int rows, int D, float eps) {
    __shared__ float red[33];
    const int nvec = D / 8;
    uint4 wv[kMaxVec];
#pragma unroll
    for (int j = 0; j < kMaxVec; j++) {
        const int i = threadIdx.x + j * NT;
        if (i < nvec) wv[j] = __ldg(reinterpret_cast<const uint4*>(w) + i);
    }
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint4* xr = reinterpret_cast<const uint4*>(x + size_t(row) * D);
        uint4 xv[kMaxVec];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < kMaxVec; j++) {
            const int i = threadIdx.x + j * NT;
            if (i < nvec) {
                xv[j] = xr[i];
                float f[8];
                unpack8(xv[j], f);
#pragma unroll
                for (int e = 0; e < 8; e++) ss += f[e] * f[e];
            }
        }
        ss = block_sum(ss, red);
        const float rms = 1.0f / sqrtf(ss / float(D) + eps);
        if (threadIdx.x == 0 && rms_out) rms_out[row] = rms;
        uint4* orow = reinterpret_cast<uint4*>(out + size_t(row) * D);
#pragma unroll
        for (int j = 0; j < kMaxVec; j++) {
            const int i = threadIdx.x + j * NT;
            if (i < nvec) {
                float f[8], g[8];
                unpack8(xv[j], f);
                unpack8(wv[j], g);
#pragma unroll
                for (int e = 0; e < 8; e++) f[e] = f[e] * rms * g[e];
                orow[i] = pack8(f);
            }
        }
    }
}

template <int NT>
__global__ void __launch_bounds__(NT) rms_norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                          const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ w,
                                                          const float* __restrict__ rms_saved,
                                                          __nv_bfloat16* __restrict__ dx,
                                                          const __nv_bfloat16* __restrict__ add_to, int rows, int D) {
    __shared__ float red[33];
    const int nvec = D / 8;
    uint4 wv[kMaxVec];
#pragma unroll
    for (int j = 0; j < kMaxVec; j++) {
        const int i = threadIdx.x + j * NT;
        if (i < nvec) wv[j] = __ldg(reinterpret_cast<const uint4*>(w) + i);
    }
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint4* xr = reinterpret_cast<const uint4*>(x + size_t(row) * D);
        const uint4* dr = reinterpret_cast<const uint4*>(dy + size_t(row) * D);
        const float rms = rms_saved[row];
        uint4 xv[kMaxVec], dv[kMaxVec];
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < kMaxVec; j++) {
            const int i = threadIdx.x + j * NT;
            if (i < nvec) {
                xv[j] = xr[i];
                dv[j] = dr[i];
                float fx[8], fd[8], fw[8];
                unpack8(xv[j], fx);
                unpack8(dv[j], fd);
                unpack8(wv[j], fw);
#pragma unroll
                for (int e = 0; e < 8; e++) dot += fd[e] * fw[e] * (fx[e] * rms);
            }
        }
        dot = block_sum(dot, red);
        const float corr = dot / float(D);
        uint4* orow = reinterpret_cast<uint4*>(dx + size_t(row) * D);
        const uint4* arow = add_to ? reinterpret_cast<const uint4*>(add_to + size_t(row) * D) : nullptr;
#pragma unroll
        for (int j = 0; j < kMaxVec; j++) {
            const int i = threadIdx.x + j * NT;
            if (i < nvec) {
                float fx[8], fd[8], fw[8], o[8];
                unpack8(xv[j], fx);
                unpack8(dv[j], fd);
                unpack8(wv[j], fw);
#pragma unroll
                for (int e = 0; e < 8; e++) o[e] = rms * (fw[e] * fd[e] - (fx[e] * rms) * corr);
                if (arow) {
                    // fused residual-gradient add: out = bf16(add_to + bf16(dx)), the two roundings of
                    // rms_norm_bwd followed by add_inplace
                    float fa[8];
                    const uint4 av = arow[i];
                    unpack8(av, fa);
#pragma unroll
                    for (int e = 0; e < 8; e++) o[e] = fa[e] + __bfloat162float(__float2bfloat16(o[e]));
                }
                orow[i] = pack8(o);
            }
        }
    }
}

// Warp-per-row variants: no block-level barrier, 8 independent rows in flight per CTA and several CTAs
// per SM, which is what keeps enough bytes in flight to approach the HBM rate.  Used when a lane can hold
// its share of the row (NV 16-byte vectors per lane, D <= 32*NV*8).
template <int NV>
__global__ void __launch_bounds__(256) rms_norm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x,
                                                                const __nv_bfloat16* __restrict__ w,
                                                                __nv_bfloat16* __restrict__ out,
                                                                float* __restrict__ rms_out, int rows, int D, float eps) {
    const int lane = threadIdx.x & 31;
    const int nvec = D / 8;
    const int wpb = blockDim.x >> 5;
    const uint4* wv = reinterpret_cast<const uint4*>(w);
    for (int row = blockIdx.x * wpb + (threadIdx.x >> 5); row < rows; row += gridDim.x * wpb) {
        const uint4* xr = reinterpret_cast<const uint4*>(x + size_t(row) * D);
        uint4 xv[NV];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const int i = lane + j * 32;
            if (i < nvec) xv[j] = xr[i];
        }
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const int i = lane + j * 32;
            if (i < nvec) {
                float f[8];
                unpack8(xv[j], f);
#pragma unroll
                for (int e = 0; e < 8; e++) ss += f[e] * f[e];
            }
        }
        ss = warp_sum(ss);
        const float rms = 1.0f / sqrtf(ss / float(D) + eps);
        if (lane == 0 && rms_out) rms_out[row] = rms;
        uint4* orow = reinterpret_cast<uint4*>(out + size_t(row) * D);
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const int i = lane + j * 32;
            if (i < nvec) {
                float f[8], g[8];
                unpack8(xv[j], f);
                unpack8(__ldg(wv + i), g);
#pragma unroll
                for (int e = 0; e < 8; e++) f[e] = f[e] * rms * g[e];
                orow[i] = pack8(f);
            }
        }
    }
}

template <int NV>
__global__ void __launch_bounds__(256) rms_norm_bwd_warp_kernel(const __nv_bfloat16* __restrict__ dy,
                                                                const __nv_bfloat16* __restrict__ x,
                                                                const __nv_bfloat16* __restrict__ w,
                                                                const float* __restrict__ rms_saved,
                                                                __nv_bfloat16* __restrict__ dx,
                                                                const __nv_bfloat16* __restrict__ add_to, int rows, int D) {
    const int lane = threadIdx.x & 31;
    const int nvec = D / 8;
    const int wpb = blockDim.x >> 5;
    const uint4* wv = reinterpret_cast<const uint4*>(w);
    for (int row = blockIdx.x * wpb + (threadIdx.x >> 5); row < rows; row += gridDim.x * wpb) {
        const uint4* xr = reinterpret_cast<const uint4*>(x + size_t(row) * D);
        const uint4* dr = reinterpret_cast<const uint4*>(dy + size_t(row) * D);
        const float rms = rms_saved[row];
        uint4 xv[NV], dv[NV];
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const int i = lane + j * 32;
            if (i < nvec) { xv[j] = xr[i]; dv[j] = dr[i]; }
        }
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const int i = lane + j * 32;
            if (i < nvec) {
                float fx[8], fd[8], fw[8];
                unpack8(xv[j], fx); unpack8(dv[j], fd); unpack8(__ldg(wv + i), fw);
#pragma unroll
                for (int e = 0; e < 8; e++) dot += fd[e] * fw[e] * (fx[e] * rms);
            }
        }
        dot = warp_sum(dot);
        const float corr = dot / float(D);
        uint4* orow = reinterpret_cast<uint4*>(dx + size_t(row) * D);
        const uint4* arow = add_to ? reinterpret_cast<const uint4*>(add_to + size_t(row) * D) : nullptr;
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const int i = lane + j * 32;
            if (i < nvec) {
                float fx[8], fd[8], fw[8], o[8];
                unpack8(xv[j], fx); unpack8(dv[j], fd); unpack8(__ldg(wv + i), fw);
#pragma unroll
                for (int e = 0; e < 8; e++) o[e] = rms * (fw[e] * fd[e] - (fx[e] * rms) * corr);
                if (arow) {
                    float fa[8];
                    const uint4 av = arow[i];
                    unpack8(av, fa);
#pragma unroll
                    for (int e = 0; e < 8; e++) o[e] = fa[e] + __bfloat162float(__float2bfloat16(o[e]));
                }
                orow[i] = pack8(o);
            }
        }
    }
}

// ── RoPE (adjacent pairs) ───────────────────────────────────────────────────
// Thread = (token, group of 4 pairs); it computes its 4 (cos, sin) once and applies them to every
// head of up to two tensors (Q and K), so the transcendental cost is amortised over the heads.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ q, int Hq, __nv_bfloat16* __restrict__ k, int Hk, int BT, int T,
                            int hd, float theta, int inverse) {
    const int gpr = hd / 8;   // 16-byte groups per head
    const long idx = blockIdx.x * long(blockDim.x) + threadIdx.x;
    if (idx >= long(BT) * gpr) return;
    const int g = int(idx % gpr);
    const int bt = int(idx / gpr);
    const int t = bt % T;
    float cs[4], sn[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int i = g * 4 + j;
        const float freq = powf(theta, -2.f * float(i) / float(hd));
        float ang = float(t) * freq;
        if (inverse) ang = -ang;
        sincosf(ang, &sn[j], &cs[j]);
    }
    for (int pass = 0; pass < 2; pass++) {
        __nv_bfloat16* base = pass == 0 ? q : k;
        const int H = pass == 0 ? Hq : Hk;
        if (!base) continue;
        uint4* row = reinterpret_cast<uint4*>(base + size_t(bt) * H * hd);
        // four heads per round: all four loads are issued before the first store (the rotation is in place, so the
        // compiler cannot hoist a load over the previous head's store by itself)
        for (int h0 = 0; h0 < H; h0 += 4) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (h0 + u < H) v[u] = row[(h0 + u) * gpr + g];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                if (h0 + u >= H) break;
                float f[8];
                unpack8(v[u], f);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float x0 = f[2 * j], x1 = f[2 * j + 1];
                    f[2 * j] = x0 * cs[j] - x1 * sn[j];
                    f[2 * j + 1] = x0 * sn[j] + x1 * cs[j];
                }
                row[(h0 + u) * gpr + g] = pack8(f);
            }
        }
    }
}

// ── SwiGLU ──────────────────────────────────────────────────────────────────
__global__ void silu_mul_fwd_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up,
                                    uint4* __restrict__ out, long nvec) {
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < nvec; i += long(gridDim.x) * blockDim.x) {
        float g[8], u[8];
        unpack8(gate[i], g);
        unpack8(up[i], u);
#pragma unroll
        for (int e = 0; e < 8; e++) g[e] = g[e] / (1.f + expf(-g[e])) * u[e];
        out[i] = pack8(g);
    }
}
__global__ void silu_mul_bwd_kernel(const uint4* __restrict__ dout, const uint4* __restrict__ gate,
                                    const uint4* __restrict__ up, uint4* __restrict__ dgate, uint4* __restrict__ dup,
                                    long nvec) {
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < nvec; i += long(gridDim.x) * blockDim.x) {
        float g[8], u[8], d[8], og[8], ou[8];
        unpack8(gate[i], g);
        unpack8(up[i], u);
        unpack8(dout[i], d);
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const float sig = 1.f / (1.f + expf(-g[e]));
            const float s = g[e] * sig;
            const float ds = sig * (1.f + g[e] * (1.f - sig));
            og[e] = d[e] * u[e] * ds;
            ou[e] = d[e] * s;
        }
        dgate[i] = pack8(og);
        dup[i] = pack8(ou);
    }
}

// ── embedding gather, adds, casts ───────────────────────────────────────────
__global__ void embed_fwd_kernel(const __nv_bfloat16* __restrict__ table, const int* __restrict__ tokens,
                                 __nv_bfloat16* __restrict__ out, int BT, int D) {
    const int nvec = D / 8;
    for (int bt = blockIdx.x; bt < BT; bt += gridDim.x) {
        const uint4* src = reinterpret_cast<const uint4*>(table + size_t(tokens[bt]) * D);
        uint4* dst = reinterpret_cast<uint4*>(out + size_t(bt) * D);
        for (int i = threadIdx.x; i < nvec; i += blockDim.x) dst[i] = __ldg(src + i);
    }
}
__global__ void add_inplace_kernel(uint4* __restrict__ out, const uint4* __restrict__ delta, long nvec) {
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < nvec; i += long(gridDim.x) * blockDim.x) {
        float a[8], b[8];
        unpack8(out[i], a);
        unpack8(delta[i], b);
#pragma unroll
        for (int e = 0; e < 8; e++) a[e] += b[e];
        out[i] = pack8(a);
    }
}
__global__ void lora_add_kernel(uint4* __restrict__ out, const uint4* __restrict__ delta, float scale, long nvec) {
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < nvec; i += long(gridDim.x) * blockDim.x) {
        float a[8], b[8];
        unpack8(out[i], a);
        unpack8(delta[i], b);
#pragma unroll
        for (int e = 0; e < 8; e++) a[e] += scale * b[e];
        out[i] = pack8(a);
    }
}
__global__ void add_bias_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ bias, long rows,
                                int D) {
    const int nvec = D / 8;
    const long total = rows * nvec;
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
        float a[8], b[8];
        uint4* p = reinterpret_cast<uint4*>(out) + i;
        unpack8(*p, a);
        unpack8(__ldg(reinterpret_cast<const uint4*>(bias) + (i % nvec)), b);
#pragma unroll
        for (int e = 0; e < 8; e++) a[e] += b[e];
        *p = pack8(a);
    }
}
__global__ void bf16_to_f32_kernel(const uint4* __restrict__ src, float4* __restrict__ dst, long nvec) {
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < nvec; i += long(gridDim.x) * blockDim.x) {
        float f[8];
        unpack8(src[i], f);
        dst[2 * i] = make_float4(f[0], f[1], f[2], f[3]);
        dst[2 * i + 1] = make_float4(f[4], f[5], f[6], f[7]);
    }
}
__global__ void f32_to_bf16_kernel(const float4* __restrict__ src, uint4* __restrict__ dst, long nvec) {
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < nvec; i += long(gridDim.x) * blockDim.x) {
        const float4 a = src[2 * i], b = src[2 * i + 1];
        const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        dst[i] = pack8(f);
    }
}
__global__ void bf16_to_f32_tail(const __nv_bfloat16* src, float* dst, long from, long n) {
    const long i = from + blockIdx.x * long(blockDim.x) + threadIdx.x;
    if (i < n) dst[i] = __bfloat162float(src[i]);
}
__global__ void f32_to_bf16_tail(const float* src, __nv_bfloat16* dst, long from, long n) {
    const long i = from + blockIdx.x * long(blockDim.x) + threadIdx.x;
    if (i < n) dst[i] = __float2bfloat16(src[i]);
}

// ── cross-entropy ───────────────────────────────────────────────────────────
// One CTA per row.  Pass 1 is an online (max, sum-exp) over the row with 16-byte loads; pass 2
// re-reads the row (an L2 hit: a row is ~300 KB) and writes dlogits = (softmax - onehot) * inv_count,
// which may alias `logits`.  Targets < 0 contribute loss = logsumexp and gradient softmax*inv_count,
// as the reference kernel does.
// `logits` and `dlogits` carry no __restrict__: the in-place call passes the same buffer for both.
__global__ void __launch_bounds__(1024) cross_entropy_kernel(const __nv_bfloat16* logits,
                                                             const int* __restrict__ targets,
                                                             float* __restrict__ loss,
                                                             __nv_bfloat16* dlogits, int V,
                                                             float inv_count) {
    __shared__ float red_m[32], red_s[32];
    __shared__ float s_lse;
    const long row = blockIdx.x;
    const uint4* L = reinterpret_cast<const uint4*>(logits + row * V);
    const int nvec = V / 8;
    float m = -FLT_MAX, s = 0.f;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        float f[8];
        unpack8(L[i], f);
        float lm = f[0];
#pragma unroll
        for (int e = 1; e < 8; e++) lm = fmaxf(lm, f[e]);
        if (lm > m) {
            s *= expf(m - lm);
            m = lm;
        }
#pragma unroll
        for (int e = 0; e < 8; e++) s += expf(f[e] - m);
    }
    // combine (m, s) pairs: warp, then block
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, m, o);
        const float os = __shfl_xor_sync(0xffffffffu, s, o);
        const float nm = fmaxf(m, om);
        s = s * expf(m - nm) + os * expf(om - nm);
        m = nm;
    }
    if (lane == 0) { red_m[w] = m; red_s[w] = s; }
    __syncthreads();
    if (w == 0) {
        m = lane < nw ? red_m[lane] : -FLT_MAX;
        s = lane < nw ? red_s[lane] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float om = __shfl_xor_sync(0xffffffffu, m, o);
            const float os = __shfl_xor_sync(0xffffffffu, s, o);
            const float nm = fmaxf(m, om);
            s = s * expf(m - nm) + os * expf(om - nm);
            m = nm;
        }
        if (lane == 0) {
            const float lse = logf(s) + m;
            const int tgt = targets[row];
            const float tl = tgt >= 0 ? __bfloat162float(logits[row * V + tgt]) : 0.f;
            loss[row] = -(tl - lse);
            s_lse = lse;
        }
    }
    __syncthreads();
    if (!dlogits) return;
    const float lse = s_lse;
    const int tgt = targets[row];
    uint4* dL = reinterpret_cast<uint4*>(dlogits + row * V);
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        float f[8];
        unpack8(L[i], f);
#pragma unroll
        for (int e = 0; e < 8; e++) {
            float p = expf(f[e] - lse);
            if (i * 8 + e == tgt) p -= 1.f;
            f[e] = p * inv_count;
        }
        dL[i] = pack8(f);
    }
}

inline unsigned grid_for(long n, int threads, const ta_ctx* ctx, int per_sm = 16) {
    long blocks = (n + threads - 1) / threads;
    long cap = long(ctx ? ctx->sm_count : 148) * per_sm;
    return unsigned(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace
}  // namespace ta

using namespace ta;

#define REQ(ctx, cond, msg) \
    do { if (!(cond)) return ta::fail((ctx), TA_ERR_INVALID, msg); } while (0)
#define ALIGNED16(p) ((reinterpret_cast<uintptr_t>(p) & 15) == 0)

extern "C" {

int ta_rms_norm_fwd(ta_ctx* ctx, const void* x, const void* w, void* out, float* rms_out, int rows, int D, float eps,
                    void* stream) {
    REQ(ctx, ctx && x && w && out && rows >= 0 && D > 0, "rms_norm_fwd: null argument or bad size");
    REQ(ctx, D % 8 == 0 && D <= 256 * kMaxVec * 8, "rms_norm_fwd: D must be a multiple of 8 and <= 16384");
    REQ(ctx, ALIGNED16(x) && ALIGNED16(w) && ALIGNED16(out), "rms_norm_fwd: pointers must be 16-byte aligned");
    if (rows == 0) return TA_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned grid = unsigned(std::min<long>(rows, long(ctx->sm_count) * 16));
    auto X = static_cast<const __nv_bfloat16*>(x);
    auto W = static_cast<const __nv_bfloat16*>(w);
    auto O = static_cast<__nv_bfloat16*>(out);
    const int nv = (D / 8 + 31) / 32;
    const unsigned wgrid = unsigned(std::min<long>((rows + 7) / 8, long(ctx->sm_count) * 8));
    if (nv <= 4)       rms_norm_fwd_warp_kernel<4><<<wgrid, 256, 0, s>>>(X, W, O, rms_out, rows, D, eps);
    else if (nv <= 8)  rms_norm_fwd_warp_kernel<8><<<wgrid, 256, 0, s>>>(X, W, O, rms_out, rows, D, eps);
    else if (nv <= 16) rms_norm_fwd_warp_kernel<16><<<wgrid, 256, 0, s>>>(X, W, O, rms_out, rows, D, eps);
    else if (D / 8 <= 128 * kMaxVec) rms_norm_fwd_kernel<128><<<grid, 128, 0, s>>>(X, W, O, rms_out, rows, D, eps);
    else                        rms_norm_fwd_kernel<256><<<grid, 256, 0, s>>>(X, W, O, rms_out, rows, D, eps);
    TA_LAUNCH_CHECK(ctx, "rms_norm_fwd_kernel");
    return TA_OK;
}

int ta_rms_norm_bwd(ta_ctx* ctx, const void* dy, const void* x, const void* w, const float* rms_saved, void* dx,
                    const void* add_to, int rows, int D, void* stream) {
    REQ(ctx, ctx && dy && x && w && rms_saved && dx && rows >= 0 && D > 0, "rms_norm_bwd: null argument or bad size");
    REQ(ctx, D % 8 == 0 && D <= 256 * kMaxVec * 8, "rms_norm_bwd: D must be a multiple of 8 and <= 16384");
    REQ(ctx, ALIGNED16(dy) && ALIGNED16(x) && ALIGNED16(w) && ALIGNED16(dx) && ALIGNED16(add_to),
        "rms_norm_bwd: pointers must be 16-byte aligned");
    if (rows == 0) return TA_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned grid = unsigned(std::min<long>(rows, long(ctx->sm_count) * 16));
    auto DY = static_cast<const __nv_bfloat16*>(dy);
    auto X = static_cast<const __nv_bfloat16*>(x);
    auto W = static_cast<const __nv_bfloat16*>(w);
    auto DX = static_cast<__nv_bfloat16*>(dx);
    auto AT = static_cast<const __nv_bfloat16*>(add_to);
    const int nv = (D / 8 + 31) / 32;
    const unsigned wgrid = unsigned(std::min<long>((rows + 7) / 8, long(ctx->sm_count) * 8));
    if (nv <= 4)       rms_norm_bwd_warp_kernel<4><<<wgrid, 256, 0, s>>>(DY, X, W, rms_saved, DX, AT, rows, D);
    else if (nv <= 8)  rms_norm_bwd_warp_kernel<8><<<wgrid, 256, 0, s>>>(DY, X, W, rms_saved, DX, AT, rows, D);
    else if (nv <= 16) rms_norm_bwd_warp_kernel<16><<<wgrid, 256, 0, s>>>(DY, X, W, rms_saved, DX, AT, rows, D);
    else if (D / 8 <= 128 * kMaxVec) rms_norm_bwd_kernel<128><<<grid, 128, 0, s>>>(DY, X, W, rms_saved, DX, AT, rows, D);
    else                        rms_norm_bwd_kernel<256><<<grid, 256, 0, s>>>(DY, X, W, rms_saved, DX, AT, rows, D);
    TA_LAUNCH_CHECK(ctx, "rms_norm_bwd_kernel");
    return TA_OK;
}

int ta_rope(ta_ctx* ctx, void* q, int Hq, void* k, int Hk, int B, int T, int head_dim, float theta, int inverse,
            void* stream) {
    REQ(ctx, ctx && (q || k) && B > 0 && T > 0, "rope: null argument or bad size");
    REQ(ctx, head_dim % 8 == 0 && head_dim > 0, "rope: head_dim must be a multiple of 8");
    REQ(ctx, ALIGNED16(q) && ALIGNED16(k), "rope: pointers must be 16-byte aligned");
    const long n = long(B) * T * (head_dim / 8);
    rope_kernel<<<unsigned((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__nv_bfloat16*>(q), q ? Hq : 0, static_cast<__nv_bfloat16*>(k), k ? Hk : 0, B * T, T, head_dim,
        theta, inverse);
    TA_LAUNCH_CHECK(ctx, "rope_kernel");
    return TA_OK;
}

int ta_silu_mul_fwd(ta_ctx* ctx, const void* gate, const void* up, void* out, long n, void* stream) {
    REQ(ctx, ctx && gate && up && out && n >= 0 && n % 8 == 0, "silu_mul_fwd: null argument or n % 8 != 0");
    REQ(ctx, ALIGNED16(gate) && ALIGNED16(up) && ALIGNED16(out), "silu_mul_fwd: pointers must be 16-byte aligned");
    if (n == 0) return TA_OK;
    silu_mul_fwd_kernel<<<grid_for(n / 8, 256, ctx), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(gate), static_cast<const uint4*>(up), static_cast<uint4*>(out), n / 8);
    TA_LAUNCH_CHECK(ctx, "silu_mul_fwd_kernel");
    return TA_OK;
}

int ta_silu_mul_bwd(ta_ctx* ctx, const void* dout, const void* gate, const void* up, void* dgate, void* dup, long n,
                    void* stream) {
    REQ(ctx, ctx && dout && gate && up && dgate && dup && n >= 0 && n % 8 == 0, "silu_mul_bwd: null argument or n % 8 != 0");
    REQ(ctx, ALIGNED16(dout) && ALIGNED16(gate) && ALIGNED16(up) && ALIGNED16(dgate) && ALIGNED16(dup),
        "silu_mul_bwd: pointers must be 16-byte aligned");
    if (n == 0) return TA_OK;
    silu_mul_bwd_kernel<<<grid_for(n / 8, 256, ctx), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(dout), static_cast<const uint4*>(gate), static_cast<const uint4*>(up),
        static_cast<uint4*>(dgate), static_cast<uint4*>(dup), n / 8);
    TA_LAUNCH_CHECK(ctx, "silu_mul_bwd_kernel");
    return TA_OK;
}

int ta_embed_fwd(ta_ctx* ctx, const void* table, const int* tokens, void* out, int BT, int D, void* stream) {
    REQ(ctx, ctx && table && tokens && out && BT >= 0 && D > 0 && D % 8 == 0, "embed_fwd: null argument or D % 8 != 0");
    REQ(ctx, ALIGNED16(table) && ALIGNED16(out), "embed_fwd: pointers must be 16-byte aligned");
    if (BT == 0) return TA_OK;
    embed_fwd_kernel<<<unsigned(std::min<long>(BT, long(ctx->sm_count) * 16)), 128, 0,
                       static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(table), tokens,
                                                             static_cast<__nv_bfloat16*>(out), BT, D);
    TA_LAUNCH_CHECK(ctx, "embed_fwd_kernel");
    return TA_OK;
}

int ta_add_inplace(ta_ctx* ctx, void* out, const void* delta, long n, void* stream) {
    REQ(ctx, ctx && out && delta && n >= 0 && n % 8 == 0, "add_inplace: null argument or n % 8 != 0");
    REQ(ctx, ALIGNED16(out) && ALIGNED16(delta), "add_inplace: pointers must be 16-byte aligned");
    if (n == 0) return TA_OK;
    add_inplace_kernel<<<grid_for(n / 8, 256, ctx), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint4*>(out), static_cast<const uint4*>(delta), n / 8);
    TA_LAUNCH_CHECK(ctx, "add_inplace_kernel");
    return TA_OK;
}

int ta_lora_add(ta_ctx* ctx, void* out, const void* delta, float scale, long n, void* stream) {
    REQ(ctx, ctx && out && delta && n >= 0 && n % 8 == 0, "lora_add: null argument or n % 8 != 0");
    REQ(ctx, ALIGNED16(out) && ALIGNED16(delta), "lora_add: pointers must be 16-byte aligned");
    if (n == 0) return TA_OK;
    lora_add_kernel<<<grid_for(n / 8, 256, ctx), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint4*>(out), static_cast<const uint4*>(delta), scale, n / 8);
    TA_LAUNCH_CHECK(ctx, "lora_add_kernel");
    return TA_OK;
}

int ta_add_bias(ta_ctx* ctx, void* out, const void* bias, long rows, int D, void* stream) {
    REQ(ctx, ctx && out && bias && rows >= 0 && D > 0 && D % 8 == 0, "add_bias: null argument or D % 8 != 0");
    REQ(ctx, ALIGNED16(out) && ALIGNED16(bias), "add_bias: pointers must be 16-byte aligned");
    if (rows == 0) return TA_OK;
    add_bias_kernel<<<grid_for(rows * (D / 8), 256, ctx), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(bias), rows, D);
    TA_LAUNCH_CHECK(ctx, "add_bias_kernel");
    return TA_OK;
}

int ta_cast_bf16_to_f32(ta_ctx* ctx, const void* src, float* dst, long n, void* stream) {
    REQ(ctx, ctx && src && dst && n >= 0, "cast_bf16_to_f32: null argument");
    REQ(ctx, ALIGNED16(src) && ALIGNED16(dst), "cast_bf16_to_f32: pointers must be 16-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const long nvec = n / 8;
    if (nvec) {
        bf16_to_f32_kernel<<<grid_for(nvec, 256, ctx), 256, 0, s>>>(static_cast<const uint4*>(src),
                                                                    reinterpret_cast<float4*>(dst), nvec);
        TA_LAUNCH_CHECK(ctx, "bf16_to_f32_kernel");
    }
    if (n % 8) {
        bf16_to_f32_tail<<<1, 32, 0, s>>>(static_cast<const __nv_bfloat16*>(src), dst, nvec * 8, n);
        TA_LAUNCH_CHECK(ctx, "bf16_to_f32_tail");
    }
    return TA_OK;
}

int ta_cast_f32_to_bf16(ta_ctx* ctx, const float* src, void* dst, long n, void* stream) {
    REQ(ctx, ctx && src && dst && n >= 0, "cast_f32_to_bf16: null argument");
    REQ(ctx, ALIGNED16(src) && ALIGNED16(dst), "cast_f32_to_bf16: pointers must be 16-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const long nvec = n / 8;
    if (nvec) {
        f32_to_bf16_kernel<<<grid_for(nvec, 256, ctx), 256, 0, s>>>(reinterpret_cast<const float4*>(src),
                                                                    static_cast<uint4*>(dst), nvec);
        TA_LAUNCH_CHECK(ctx, "f32_to_bf16_kernel");
    }
    if (n % 8) {
        f32_to_bf16_tail<<<1, 32, 0, s>>>(src, static_cast<__nv_bfloat16*>(dst), nvec * 8, n);
        TA_LAUNCH_CHECK(ctx, "f32_to_bf16_tail");
    }
    return TA_OK;
}

int ta_cross_entropy_fwd(ta_ctx* ctx, const void* logits, const int* targets, float* loss_out, void* dlogits, int rows,
                         int V, float inv_count, void* stream) {
    REQ(ctx, ctx && logits && targets && loss_out && rows >= 0 && V > 0, "cross_entropy_fwd: null argument or bad size");
    REQ(ctx, V % 8 == 0, "cross_entropy_fwd: V must be a multiple of 8");
    REQ(ctx, ALIGNED16(logits) && ALIGNED16(dlogits), "cross_entropy_fwd: pointers must be 16-byte aligned");
    if (rows == 0) return TA_OK;
    const int threads = V / 8 >= 1024 ? 1024 : std::max(32, ((V / 8 + 31) / 32) * 32);
    cross_entropy_kernel<<<rows, threads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(logits), targets, loss_out, static_cast<__nv_bfloat16*>(dlogits), V,
        inv_count);
    TA_LAUNCH_CHECK(ctx, "cross_entropy_kernel");
    return TA_OK;
}

}  // extern "C"
