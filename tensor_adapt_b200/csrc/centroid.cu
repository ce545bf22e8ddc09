// Centroid Accumulator on the device: per-token gradient-norm-weighted sum of hidden states
// (C = sum_t h_t * ||g_t||), and the k-means merge of snapshot vectors.
//
// Accumulation is HBM-bound: it reads h[BT,D] and g[BT,D] once (2*BT*D*2 bytes) and replaces the
// reference's per-layer round trip of four [BT,D] FP32 copies over PCIe plus a scalar CPU loop.
// Two modes:
//   TA_CENTROID_INTENDED  acc[d] += h[t,d]*||g[t,:]||, weight += ||g[t,:]||   (the documented formula)
//   TA_CENTROID_ASBUILT   what the shipped trainer computes after it re-reads FP32 buffers through a
//                         BF16 pointer: pseudo-row u = 0..BT-1 covers token u/2, half u%2 of the row;
//                         gamma_u = ||g[tok, half*D/2 : (half+1)*D/2]||, acc[2m+1] += h[tok, half*D/2+m]*gamma_u.
// Both use a two-stage, fixed-order reduction (bit-identical from run to run).
//
// The k-means kernels keep the reference's FP32 operation order (no FMA contraction, sequential sums)
// so cluster assignments and centres are bit-exact against the CPU implementation.
#include <algorithm>

#include "ctx.h"
#include "ptx.cuh"

namespace ta {
namespace {

constexpr int kRows = 32;      // token rows per CTA
constexpr int kThreads = 256;
constexpr int kColVec = 4;     // 16-byte column vectors per thread: D <= 256*4*8 = 8192

__device__ __forceinline__ void unpack8c(const uint4& u, float (&f)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 t = unpack_bf16x2(w[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

// partial[cta][0..D) = sum over the CTA's rows of h[row][j] * gamma(row, half(j));  partial_w[cta] = sum gamma
__global__ void __launch_bounds__(kThreads) centroid_partial_kernel(const __nv_bfloat16* __restrict__ h,
                                                                    const __nv_bfloat16* __restrict__ g, int rows,
                                                                    int pseudo_rows, int D, int asbuilt,
                                                                    float* __restrict__ partial,
                                                                    float* __restrict__ partial_w) {
    __shared__ float gam[kRows][2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r0 = blockIdx.x * kRows;
    const int nvec = D / 8, half_vec = nvec / 2;
    // phase A: one warp per row computes the row's gradient norm(s)
    for (int rl = warp; rl < kRows; rl += kThreads / 32) {
        const int row = r0 + rl;
        float s0 = 0.f, s1 = 0.f;
        if (row < rows) {
            const uint4* gr = reinterpret_cast<const uint4*>(g + size_t(row) * D);
            for (int i = lane; i < nvec; i += 32) {
                float f[8];
                unpack8c(gr[i], f);
                float s = 0.f;
#pragma unroll
                for (int e = 0; e < 8; e++) s += f[e] * f[e];
                if (asbuilt && i >= half_vec) s1 += s; else s0 += s;
            }
        }
        s0 = warp_sum(s0);
        s1 = warp_sum(s1);
        if (lane == 0) {
            if (!asbuilt) {
                gam[rl][0] = gam[rl][1] = sqrtf(s0);
            } else {
                // pseudo-rows 2*row and 2*row+1 exist only while they are < pseudo_rows
                gam[rl][0] = (2 * row < pseudo_rows) ? sqrtf(s0) : 0.f;
                gam[rl][1] = (2 * row + 1 < pseudo_rows) ? sqrtf(s1) : 0.f;
            }
        }
    }
    __syncthreads();
    // phase B: column sums, coalesced 16-byte loads along the row
    float acc[kColVec][8];
#pragma unroll
    for (int j = 0; j < kColVec; j++)
#pragma unroll
        for (int e = 0; e < 8; e++) acc[j][e] = 0.f;
    const int nr = min(kRows, rows - r0);
    for (int rl = 0; rl < nr; rl++) {
        const uint4* hr = reinterpret_cast<const uint4*>(h + size_t(r0 + rl) * D);
        const float g0 = gam[rl][0], g1 = gam[rl][1];
#pragma unroll
        for (int j = 0; j < kColVec; j++) {
            const int i = threadIdx.x + j * kThreads;
            if (i < nvec) {
                float f[8];
                unpack8c(hr[i], f);
                const float gm = (asbuilt && i >= half_vec) ? g1 : g0;
#pragma unroll
                for (int e = 0; e < 8; e++) acc[j][e] += f[e] * gm;
            }
        }
    }
    float* out = partial + size_t(blockIdx.x) * D;
#pragma unroll
    for (int j = 0; j < kColVec; j++) {
        const int i = threadIdx.x + j * kThreads;
        if (i < nvec) {
            *reinterpret_cast<float4*>(out + i * 8) = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
            *reinterpret_cast<float4*>(out + i * 8 + 4) = make_float4(acc[j][4], acc[j][5], acc[j][6], acc[j][7]);
        }
    }
    if (threadIdx.x == 0) {
        float w = 0.f;
        for (int rl = 0; rl < nr; rl++) w += asbuilt ? gam[rl][0] + gam[rl][1] : gam[rl][0];
        partial_w[blockIdx.x] = w;
    }
}

// Warp-per-row variant for D <= 32*NV*8: a warp keeps its 1/32 slice of the accumulator in registers
// (NV 16-byte vectors per lane), reads a row of g (norm) and the same row of h with every load of the row
// in flight at once, and walks rows warp + k*warps-in-grid; the warps of a CTA are combined in warp order.
template <int NV>
__global__ void __launch_bounds__(kThreads) centroid_partial_warp_kernel(const __nv_bfloat16* __restrict__ h,
                                                                         const __nv_bfloat16* __restrict__ g, int rows,
                                                                         int pseudo_rows, int D, int asbuilt,
                                                                         float* __restrict__ partial,
                                                                         float* __restrict__ partial_w) {
    constexpr int kWarps = kThreads / 32;
    __shared__ float red[kWarps - 1][32 * 8 + 1];
    __shared__ float wsum[kWarps];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nvec = D / 8, half_vec = nvec / 2;
    float acc[NV][8];
#pragma unroll
    for (int j = 0; j < NV; j++)
#pragma unroll
        for (int e = 0; e < 8; e++) acc[j][e] = 0.f;
    float wacc = 0.f;
    for (int row = blockIdx.x * kWarps + warp; row < rows; row += gridDim.x * kWarps) {
        const uint4* gr = reinterpret_cast<const uint4*>(g + size_t(row) * D);
        const uint4* hr = reinterpret_cast<const uint4*>(h + size_t(row) * D);
        uint4 gv[NV], hv[NV];
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const int i = lane + 32 * j;
            gv[j] = i < nvec ? gr[i] : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const int i = lane + 32 * j;
            hv[j] = i < nvec ? hr[i] : make_uint4(0, 0, 0, 0);
        }
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int j = 0; j < NV; j++) {
            float f[8];
            unpack8c(gv[j], f);
            float s = 0.f;
#pragma unroll
            for (int e = 0; e < 8; e++) s += f[e] * f[e];
            if (asbuilt && lane + 32 * j >= half_vec) s1 += s; else s0 += s;
        }
        s0 = warp_sum(s0);
        s1 = warp_sum(s1);
        float g0, g1;
        if (!asbuilt) {
            g0 = g1 = sqrtf(s0);
            wacc += g0;
        } else {
            g0 = (2 * row < pseudo_rows) ? sqrtf(s0) : 0.f;
            g1 = (2 * row + 1 < pseudo_rows) ? sqrtf(s1) : 0.f;
            wacc += g0 + g1;
        }
#pragma unroll
        for (int j = 0; j < NV; j++) {
            float f[8];
            unpack8c(hv[j], f);
            const float gm = (asbuilt && lane + 32 * j >= half_vec) ? g1 : g0;
#pragma unroll
            for (int e = 0; e < 8; e++) acc[j][e] += f[e] * gm;
        }
    }
    // combine the CTA's warps in warp order, one vector slot at a time (bounded shared memory)
    float* out = partial + size_t(blockIdx.x) * D;
    if (lane == 0) wsum[warp] = wacc;
#pragma unroll
    for (int j = 0; j < NV; j++) {
        __syncthreads();
        if (warp > 0)
#pragma unroll
            for (int e = 0; e < 8; e++) red[warp - 1][lane * 8 + e] = acc[j][e];
        __syncthreads();
        if (warp == 0) {
            const int i = lane + 32 * j;
            float t[8];
#pragma unroll
            for (int e = 0; e < 8; e++) {
                t[e] = acc[j][e];
                for (int w = 0; w < kWarps - 1; w++) t[e] += red[w][lane * 8 + e];
            }
            if (i < nvec) {
                *reinterpret_cast<float4*>(out + i * 8) = make_float4(t[0], t[1], t[2], t[3]);
                *reinterpret_cast<float4*>(out + i * 8 + 4) = make_float4(t[4], t[5], t[6], t[7]);
            }
        }
    }
    if (threadIdx.x == 0) {
        float w = 0.f;
        for (int k = 0; k < kWarps; k++) w += wsum[k];
        partial_w[blockIdx.x] = w;
    }
}

// acc[d] += sum_b partial[b][d] in a fixed order: thread (x, y) sums blocks y, y+8, ... for column x, the
// eight partial sums are then added in y order.
__global__ void __launch_bounds__(256) centroid_reduce_kernel(const float* __restrict__ partial,
                                                              const float* __restrict__ partial_w, int nblocks, int D,
                                                              int asbuilt, float* __restrict__ acc,
                                                              float* __restrict__ weight) {
    __shared__ float part[8][33];
    const int x = threadIdx.x & 31, y = threadIdx.x >> 5;
    const int d = blockIdx.x * 32 + x;          // source column (as-built: m of the first half)
    const int ncol = asbuilt ? D / 2 : D;
    float s = 0.f;
    if (d < ncol) {
        for (int b = y; b < nblocks; b += 8) {
            const float* pr = partial + size_t(b) * D;
            s += asbuilt ? pr[d] + pr[D / 2 + d] : pr[d];
        }
    }
    part[y][x] = s;
    __syncthreads();
    if (y == 0 && d < ncol) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 8; k++) t += part[k][x];
        acc[asbuilt ? 2 * d + 1 : d] += t;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        float w = 0.f;
        for (int b = 0; b < nblocks; b++) w += partial_w[b];
        *weight += w;
    }
}

// ── k-means (bit-exact with the sequential FP32 host loop) ──────────────────

__global__ void kmeans_init_kernel(const float* __restrict__ vec, int N, int D, int k, float* __restrict__ centers,
                                   int* __restrict__ assign) {
    const long i = blockIdx.x * long(blockDim.x) + threadIdx.x;
    if (i < long(k) * D) {
        const int ki = int(i / D), d = int(i - long(ki) * D);
        centers[i] = vec[size_t((long(ki) * N) / k) * D + d];
    }
    if (i < N) assign[i] = 0;
}

// one thread per (vector, centre): d = (((0 + v0*v0) + v1*v1) + ...) with separately rounded mul and add
__global__ void kmeans_dist_kernel(const float* __restrict__ vec, const float* __restrict__ centers, int N, int D, int k,
                                   float* __restrict__ dist) {
    const long i = blockIdx.x * long(blockDim.x) + threadIdx.x;
    if (i >= long(N) * k) return;
    const int n = int(i / k), ki = int(i - long(n) * k);
    const float* x = vec + size_t(n) * D;
    const float* c = centers + size_t(ki) * D;
    float d = 0.f;
    for (int j = 0; j < D; j++) {
        const float v = __fsub_rn(x[j], c[j]);
        d = __fadd_rn(d, __fmul_rn(v, v));
    }
    dist[i] = d;
}

__global__ void kmeans_assign_kernel(const float* __restrict__ dist, int N, int k, int* __restrict__ assign,
                                     int* __restrict__ changed) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    float best = 1e38f;
    int bk = 0;
    for (int ki = 0; ki < k; ki++) {
        const float d = dist[size_t(n) * k + ki];
        if (d < best) { best = d; bk = ki; }   // strict '<': the lowest index wins ties
    }
    if (assign[n] != bk) {
        assign[n] = bk;
        atomicExch(changed, 1);
    }
}

// one thread per (centre, coordinate): sequential sum over the members in vector order, then c /= count
__global__ void kmeans_update_kernel(const float* __restrict__ vec, const int* __restrict__ assign, int N, int D, int k,
                                     float* __restrict__ centers) {
    const long i = blockIdx.x * long(blockDim.x) + threadIdx.x;
    if (i >= long(k) * D) return;
    const int ki = int(i / D), d = int(i - long(ki) * D);
    float c = 0.f;
    int count = 0;
    for (int n = 0; n < N; n++) {
        if (assign[n] == ki) {
            c = __fadd_rn(c, vec[size_t(n) * D + d]);
            count++;
        }
    }
    centers[i] = count > 0 ? __fdiv_rn(c, float(count)) : 0.f;
}

// ── seeded k-means++ start and ranking by gradient mass (no reference code: README.md:73-79) ──

// squared distance to the newest centre, same FP32 order as kmeans_dist_kernel; keeps the running minimum
__global__ void kmeans_pp_dist_kernel(const float* __restrict__ vec, int N, int D, const int* __restrict__ chosen, int j,
                                      float* __restrict__ d2) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    const float* x = vec + size_t(n) * D;
    const float* c = vec + size_t(chosen[j]) * D;
    float d = 0.f;
    for (int i = 0; i < D; i++) {
        const float v = __fsub_rn(x[i], c[i]);
        d = __fadd_rn(d, __fmul_rn(v, v));
    }
    d2[n] = j == 0 ? d : fminf(d2[n], d);
}

// next centre: first index whose FP64 running sum of d2 exceeds u * total (one thread: the running
// sum is order-dependent and N is the number of snapshots, not a hot loop)
__global__ void kmeans_pp_pick_kernel(const float* __restrict__ d2, int N, double u, int* __restrict__ chosen, int j) {
    if (blockIdx.x || threadIdx.x) return;
    double total = 0.0;
    for (int n = 0; n < N; n++) total = __dadd_rn(total, double(d2[n]));
    const double r = __dmul_rn(u, total);
    double run = 0.0;
    int pick = N - 1;
    for (int n = 0; n < N; n++) {
        run = __dadd_rn(run, double(d2[n]));
        if (run > r) { pick = n; break; }
    }
    chosen[j] = pick;
}

__global__ void kmeans_gather_kernel(const float* __restrict__ vec, int N, int D, int k, const int* __restrict__ chosen,
                                     float* __restrict__ centers, int* __restrict__ assign) {
    const long i = blockIdx.x * long(blockDim.x) + threadIdx.x;
    if (i < long(k) * D) {
        const int ki = int(i / D), d = int(i - long(ki) * D);
        centers[i] = vec[size_t(chosen[ki]) * D + d];
    }
    if (i < N) assign[i] = 0;
}

// per-cluster FP64 mass in vector order, then a stable descending order of the clusters (k is small)
__global__ void kmeans_rank_kernel(const int* __restrict__ assign, const float* __restrict__ mass, int N, int k,
                                   double* __restrict__ tot, int* __restrict__ order, int* __restrict__ inverse) {
    const int ki = threadIdx.x;
    if (ki < k) {
        double t = 0.0;
        for (int n = 0; n < N; n++)
            if (assign[n] == ki) t = __dadd_rn(t, mass ? double(mass[n]) : 1.0);
        tot[ki] = t;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 0; i < k; i++) order[i] = i;
        for (int i = 1; i < k; i++) {   // insertion sort: equal masses keep their index order
            const int o = order[i];
            int j = i - 1;
            while (j >= 0 && tot[order[j]] < tot[o]) { order[j + 1] = order[j]; j--; }
            order[j + 1] = o;
        }
        for (int i = 0; i < k; i++) inverse[order[i]] = i;
    }
}

__global__ void kmeans_permute_kernel(const float* __restrict__ centers_in, const double* __restrict__ tot_in, int D, int k, int N,
                                      const int* __restrict__ order, const int* __restrict__ inverse,
                                      float* __restrict__ centers_out, double* __restrict__ tot_out, int* __restrict__ assign) {
    const long i = blockIdx.x * long(blockDim.x) + threadIdx.x;
    if (i < long(k) * D) {
        const int ki = int(i / D), d = int(i - long(ki) * D);
        centers_out[i] = centers_in[size_t(order[ki]) * D + d];
    }
    if (i < k && tot_out) tot_out[i] = tot_in[order[i]];
    if (i < N) assign[i] = inverse[assign[i]];
}

}  // namespace
}  // namespace ta

using namespace ta;

extern "C" {

int ta_centroid_accumulate(ta_ctx* ctx, int mode, const void* hidden, const void* grad_signal, int BT, int D, float* acc,
                           float* weight, void* stream) {
    if (!ctx || !hidden || !grad_signal || !acc || !weight || BT < 0 || D <= 0)
        return fail(ctx, TA_ERR_INVALID, "centroid_accumulate: null argument or bad size");
    if (mode != TA_CENTROID_INTENDED && mode != TA_CENTROID_ASBUILT)
        return fail(ctx, TA_ERR_INVALID, "centroid_accumulate: unknown mode");
    const int asbuilt = mode == TA_CENTROID_ASBUILT;
    if (D % (asbuilt ? 16 : 8) != 0 || D > kThreads * kColVec * 8)
        return fail(ctx, TA_ERR_INVALID, "centroid_accumulate: D must be a multiple of 8 (16 as-built) and <= 8192");
    if ((reinterpret_cast<uintptr_t>(hidden) & 15) || (reinterpret_cast<uintptr_t>(grad_signal) & 15))
        return fail(ctx, TA_ERR_INVALID, "centroid_accumulate: pointers must be 16-byte aligned");
    if (BT == 0) return TA_OK;
    // as-built reads only the first BT*D BF16 elements of the FP32 buffers = tokens 0 .. ceil(BT/2)-1
    const int rows = asbuilt ? (BT + 1) / 2 : BT;
    const int nv = (D / 8 + 31) / 32;   // 16-byte vectors per lane in the warp-per-row kernel
    const bool warp_rows = nv <= 16;
    const int blocks = warp_rows ? std::min((rows + kThreads / 32 - 1) / (kThreads / 32), (nv <= 8 ? 2 : 1) * ctx->sm_count)
                                 : (rows + kRows - 1) / kRows;
    void* ws = nullptr;
    if (int rc = get_workspace(ctx, size_t(blocks) * (D + 1) * sizeof(float), &ws)) return rc;
    float* partial = static_cast<float*>(ws);
    float* partial_w = partial + size_t(blocks) * D;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const __nv_bfloat16* hb = static_cast<const __nv_bfloat16*>(hidden);
    const __nv_bfloat16* gb = static_cast<const __nv_bfloat16*>(grad_signal);
    if (!warp_rows) centroid_partial_kernel<<<blocks, kThreads, 0, s>>>(hb, gb, rows, BT, D, asbuilt, partial, partial_w);
    else if (nv <= 4) centroid_partial_warp_kernel<4><<<blocks, kThreads, 0, s>>>(hb, gb, rows, BT, D, asbuilt, partial, partial_w);
    else if (nv <= 8) centroid_partial_warp_kernel<8><<<blocks, kThreads, 0, s>>>(hb, gb, rows, BT, D, asbuilt, partial, partial_w);
    else centroid_partial_warp_kernel<16><<<blocks, kThreads, 0, s>>>(hb, gb, rows, BT, D, asbuilt, partial, partial_w);
    TA_LAUNCH_CHECK(ctx, "centroid_partial_kernel");
    const int ncol = asbuilt ? D / 2 : D;
    centroid_reduce_kernel<<<(ncol + 31) / 32, 256, 0, s>>>(partial, partial_w, blocks, D, asbuilt, acc, weight);
    TA_LAUNCH_CHECK(ctx, "centroid_reduce_kernel");
    return TA_OK;
}

// Lloyd passes from the centres already in `centers` (assign starts at 0 everywhere)
static int kmeans_lloyd(ta_ctx* ctx, const float* vectors, int N, int D, int k, int max_iters, float* centers, int* assign,
                        int* changed, float* dist, int* passes_out, cudaStream_t s) {
    int passes = 0;
    for (int it = 0; it < max_iters; it++) {
        passes++;
        TA_CUDA(ctx, cudaMemsetAsync(changed, 0, sizeof(int), s));
        kmeans_dist_kernel<<<unsigned((long(N) * k + 127) / 128), 128, 0, s>>>(vectors, centers, N, D, k, dist);
        TA_LAUNCH_CHECK(ctx, "kmeans_dist_kernel");
        kmeans_assign_kernel<<<(N + 127) / 128, 128, 0, s>>>(dist, N, k, assign, changed);
        TA_LAUNCH_CHECK(ctx, "kmeans_assign_kernel");
        int h = 0;
        TA_CUDA(ctx, cudaMemcpyAsync(&h, changed, sizeof(int), cudaMemcpyDeviceToHost, s));
        TA_CUDA(ctx, cudaStreamSynchronize(s));
        if (!h) break;
        kmeans_update_kernel<<<unsigned((long(k) * D + 127) / 128), 128, 0, s>>>(vectors, assign, N, D, k, centers);
        TA_LAUNCH_CHECK(ctx, "kmeans_update_kernel");
    }
    if (passes_out) *passes_out = passes;
    return TA_OK;
}

int ta_kmeans_merge(ta_ctx* ctx, const float* vectors, int N, int D, int k, int max_iters, float* centers, int* assign,
                    int* k_out, int* passes_out, void* stream) {
    if (!ctx || !vectors || !centers || !assign || N <= 0 || D <= 0 || k <= 0 || max_iters < 0)
        return fail(ctx, TA_ERR_INVALID, "kmeans_merge: null argument or bad size");
    k = std::min(k, N);
    if (k_out) *k_out = k;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    void* ws = nullptr;
    if (int rc = get_workspace(ctx, size_t(N) * k * sizeof(float) + 256, &ws)) return rc;
    int* changed = static_cast<int*>(ws);
    float* dist = reinterpret_cast<float*>(static_cast<char*>(ws) + 256);
    const long ninit = std::max<long>(long(k) * D, N);
    kmeans_init_kernel<<<unsigned((ninit + 255) / 256), 256, 0, s>>>(vectors, N, D, k, centers, assign);
    TA_LAUNCH_CHECK(ctx, "kmeans_init_kernel");
    return kmeans_lloyd(ctx, vectors, N, D, k, max_iters, centers, assign, changed, dist, passes_out, s);
}

int ta_kmeans_merge_ex(ta_ctx* ctx, const float* vectors, const float* mass, int N, int D, int k, int max_iters, int init_mode,
                       unsigned long long seed, int rank_by_mass, float* centers, int* assign, double* cluster_mass,
                       int* init_index, int* k_out, int* passes_out, void* stream) {
    if (!ctx || !vectors || !centers || !assign || N <= 0 || D <= 0 || k <= 0 || max_iters < 0 ||
        (init_mode != TA_KMEANS_INIT_EVEN && init_mode != TA_KMEANS_INIT_PLUSPLUS))
        return fail(ctx, TA_ERR_INVALID, "kmeans_merge_ex: null argument, bad size or unknown init mode");
    k = std::min(k, N);
    if (k > 1024) return fail(ctx, TA_ERR_UNSUPPORTED, "kmeans_merge_ex: at most 1024 clusters");
    if (k_out) *k_out = k;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // workspace: changed flag | dist [N,k] | d2 [N] | chosen [k] | order [k] | inverse [k] | tot [k] f64 | centres copy [k,D]
    auto al = [](size_t x) { return (x + 255) & ~size_t(255); };
    const size_t o_dist = 256, o_d2 = o_dist + al(size_t(N) * k * 4), o_ch = o_d2 + al(size_t(N) * 4), o_ord = o_ch + al(size_t(k) * 4),
                 o_inv = o_ord + al(size_t(k) * 4), o_tot = o_inv + al(size_t(k) * 4), o_cc = o_tot + al(size_t(k) * 8),
                 total = o_cc + al(size_t(k) * D * 4);
    void* ws = nullptr;
    if (int rc = get_workspace(ctx, total, &ws)) return rc;
    char* w = static_cast<char*>(ws);
    int* changed = reinterpret_cast<int*>(w);
    float* dist = reinterpret_cast<float*>(w + o_dist);
    float* d2 = reinterpret_cast<float*>(w + o_d2);
    int* chosen = reinterpret_cast<int*>(w + o_ch);
    int* order = reinterpret_cast<int*>(w + o_ord);
    int* inverse = reinterpret_cast<int*>(w + o_inv);
    double* tot = reinterpret_cast<double*>(w + o_tot);
    float* ccopy = reinterpret_cast<float*>(w + o_cc);
    const long ninit = std::max<long>(long(k) * D, N);
    if (init_mode == TA_KMEANS_INIT_EVEN) {
        kmeans_init_kernel<<<unsigned((ninit + 255) / 256), 256, 0, s>>>(vectors, N, D, k, centers, assign);
        TA_LAUNCH_CHECK(ctx, "kmeans_init_kernel");
    } else {
        // 64-bit LCG (Knuth's MMIX constants), 53-bit uniforms; the draws happen on the host, the
        // distances and the picks on the device with no synchronisation in between
        unsigned long long st = seed * 6364136223846793005ull + 1442695040888963407ull;
        auto next_u = [&]() {
            st = st * 6364136223846793005ull + 1442695040888963407ull;
            return double(st >> 11) / 9007199254740992.0;
        };
        const int first = int(next_u() * N) % N;
        TA_CUDA(ctx, cudaMemcpyAsync(chosen, &first, sizeof(int), cudaMemcpyHostToDevice, s));
        TA_CUDA(ctx, cudaStreamSynchronize(s));   // `first` is a stack variable
        for (int j = 1; j < k; j++) {
            kmeans_pp_dist_kernel<<<(N + 127) / 128, 128, 0, s>>>(vectors, N, D, chosen, j - 1, d2);
            TA_LAUNCH_CHECK(ctx, "kmeans_pp_dist_kernel");
            kmeans_pp_pick_kernel<<<1, 32, 0, s>>>(d2, N, next_u(), chosen, j);
            TA_LAUNCH_CHECK(ctx, "kmeans_pp_pick_kernel");
        }
        kmeans_gather_kernel<<<unsigned((ninit + 255) / 256), 256, 0, s>>>(vectors, N, D, k, chosen, centers, assign);
        TA_LAUNCH_CHECK(ctx, "kmeans_gather_kernel");
        if (init_index) TA_CUDA(ctx, cudaMemcpyAsync(init_index, chosen, size_t(k) * sizeof(int), cudaMemcpyDeviceToDevice, s));
    }
    if (int rc = kmeans_lloyd(ctx, vectors, N, D, k, max_iters, centers, assign, changed, dist, passes_out, s)) return rc;
    if (rank_by_mass || cluster_mass) {
        kmeans_rank_kernel<<<1, 1024, 0, s>>>(assign, mass, N, k, tot, order, inverse);
        TA_LAUNCH_CHECK(ctx, "kmeans_rank_kernel");
        if (rank_by_mass) {
            TA_CUDA(ctx, cudaMemcpyAsync(ccopy, centers, size_t(k) * D * 4, cudaMemcpyDeviceToDevice, s));
            kmeans_permute_kernel<<<unsigned((ninit + 255) / 256), 256, 0, s>>>(ccopy, tot, D, k, N, order, inverse, centers, cluster_mass,
                                                                               assign);
            TA_LAUNCH_CHECK(ctx, "kmeans_permute_kernel");
        } else {
            TA_CUDA(ctx, cudaMemcpyAsync(cluster_mass, tot, size_t(k) * 8, cudaMemcpyDeviceToDevice, s));
        }
    }
    return TA_OK;
}

}  // extern "C"
