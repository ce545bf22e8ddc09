// Causal GQA attention for sm_100a, flash style: no [T,T] matrix ever reaches HBM, only
// LSE[B,Hq,T] is saved for the backward.  All contractions run on tcgen05 with TMEM accumulators,
// operands arrive by TMA into 128B-swizzled shared memory.
//
// Layouts (the reference's, src/backend/cuda/ops.cu:440-458): Q, O, dO, dQ are [B*T, Hq*hd],
// K, V, dK, dV are [B*T, Hkv*hd], heads interleaved in the feature dimension; hd is 64 or 128.
//
//   attn_fwd_kernel     CTA = (128 query rows, head, batch); S = Q.K^T and O_j = P.V per 128-key tile
//   attn_delta_kernel   delta[b,h,t] = sum_d dO*O
//   attn_bwd_dq_kernel  CTA = (128 query rows, head, batch); dQ accumulates in TMEM over 128-key tiles
//   attn_bwd_dkv_kernel CTA = (128 key rows, KV head, batch); dK, dV accumulate in TMEM over all query
//                       tiles AND all query heads of the GQA group, so no atomics are needed
//
// 320 threads per CTA: warp 0 = TMA producer, warp 1 = MMA issuer (one elected thread), warps 2-9 = two
// groups of four softmax / element-wise warps (one thread per tile row = TMEM lane) that work on
// alternating key tiles / sub-tiles.  In the backward kernels the second contractions read their A operand
// (dS, P^T, dS^T) straight from tensor memory.  Every wait is bounded.
#include <algorithm>
#include <cmath>

#include "ctx.h"
#include "ptx.cuh"

namespace ta {
namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct AttnParams {
    CUtensorMap tmQ, tmK, tmV, tmdO;          // boxes of 128 rows
    CUtensorMap tmQ64, tmdO64;                // boxes of 64 rows (query sub-tiles of the dK/dV kernel)
    CUtensorMap tmOut;                        // fwd: O, dq: dQ; box of 32 rows x 64 columns (one warp's share of a tile)
    __nv_bfloat16* out;        // fwd: O ; dq: dQ
    __nv_bfloat16* out2;       // dkv: dK
    __nv_bfloat16* out3;       // dkv: dV
    float* lse;                // [B*Hq*T]
    const float* delta;        // [B*Hq*T]
    int kv_parts;              // dkv: CTAs per (key tile, KV head, batch), each over a share of the group's query heads
    float* part;               // dkv, kv_parts > 1: FP32 partial sums [2 (dK, dV)][kv_parts][B*T][Hkv*hd]
    int B, T, Hq, Hkv;
    float scale, scale_log2;
    int* status;
};

// byte offset of element (row, col) of a BF16 operand stored as K-major 64-column chunks of
// [128 rows][128 B] with the 128-byte swizzle (16-byte units XOR row%8)
__device__ __forceinline__ uint32_t kmajor_off(int row, int col) {
    const int chunk = col >> 6, c = col & 63;
    return uint32_t(chunk) * 16384u + uint32_t(row) * 128u + uint32_t(((c >> 3) ^ (row & 7)) << 4) + uint32_t(c & 7) * 2u;
}

template <int HD>
struct Tile {
    static constexpr int NC = HD / 64;
    static constexpr uint32_t BYTES = NC * 16384u;     // [128 rows][HD]
    static constexpr uint32_t BYTES64 = NC * 8192u;    // [64 rows][HD]
};

// The MMA-issuing thread is a serial resource: 16-24 MMAs per tile iteration.  Descriptors are therefore
// built once per buffer and advanced with a single 64-bit add per MMA (the start-address field counts
// 16-byte units; shared-memory addresses stay below 256 KB, so the add never carries out of the field).
__device__ __forceinline__ uint64_t desc_k(uint32_t saddr) { return smem_desc_sw128(saddr, 16, 1024); }
__device__ __forceinline__ uint64_t desc_mn(uint32_t saddr, uint32_t chunk_bytes) {
    return smem_desc_sw128(saddr, chunk_bytes, 1024);
}

// D[128, N] (+)= A[128, HD] . B[N, HD]^T, both K-major, NC chunks of a_chunk / b_chunk bytes
template <int HD, int N>
__device__ __forceinline__ void mma_kk(uint32_t d_tmem, uint64_t a_desc, uint32_t a_chunk, uint64_t b_desc,
                                       uint32_t b_chunk, bool accumulate) {
    constexpr uint32_t idesc = umma_idesc_bf16(128, N, false, false);
#pragma unroll
    for (int c = 0; c < Tile<HD>::NC; c++)
#pragma unroll
        for (int ki = 0; ki < 4; ki++)
            umma_bf16(d_tmem, a_desc + ((c * a_chunk + ki * 32) >> 4), b_desc + ((c * b_chunk + ki * 32) >> 4), idesc,
                      (accumulate || c || ki) ? 1u : 0u);
}

// D[128, HD] (+)= A[128, KT] . B[KT (k), HD (n)]: A K-major (64-column chunks 16384 B apart), B a
// [KT rows][HD] tile read MN-major (b_desc made by desc_mn with the n-chunk stride; 16 k-rows = 2048 B)
template <int HD, int KT>
__device__ __forceinline__ void mma_kmn(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, bool accumulate) {
    constexpr uint32_t idesc = umma_idesc_bf16(128, HD, false, true);
#pragma unroll
    for (int ks = 0; ks < KT / 16; ks++)
        umma_bf16(d_tmem, a_desc + (((ks >> 2) * 16384 + (ks & 3) * 32) >> 4), b_desc + ((ks * 2048) >> 4), idesc,
                  (accumulate || ks) ? 1u : 0u);
}

// D[128, HD] (+)= A[128, KT] . B[KT (k), HD (n)] with A read from TENSOR MEMORY: BF16 packed two per
// 32-bit column (column c of the lane holds k = 2c and 2c+1), so a K = 16 step advances eight columns;
// B as in mma_kmn.  Halves the shared-memory operand traffic of the contraction and needs no P / dS tile
// in shared memory at all.
template <int HD, int KT>
__device__ __forceinline__ void mma_tmn(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, bool accumulate) {
    constexpr uint32_t idesc = umma_idesc_bf16(128, HD, false, true);
#pragma unroll
    for (int ks = 0; ks < KT / 16; ks++)
        umma_bf16_ts(d_tmem, a_tmem + ks * 8, b_desc + ((ks * 2048) >> 4), idesc, (accumulate || ks) ? 1u : 0u);
}

template <int HD>
__device__ __forceinline__ void load_tile(uint8_t* dst, uint32_t chunk_bytes, const CUtensorMap* tm, uint64_t* bar,
                                          int col0, int row0) {
#pragma unroll
    for (int c = 0; c < Tile<HD>::NC; c++) tma_load_2d(dst + c * chunk_bytes, tm, bar, col0 + 64 * c, row0);
}

// Output tiles leave through a 4 KB staging tile per warp (32 rows x 128 B in the 128-byte-swizzled layout of a
// {64, 32} TMA box) and ONE bulk tensor store, instead of 8 x 32 scattered 16-byte stores per thread row.
// Only for tiles that lie wholly inside their sequence: a bulk store clips at the end of the tensor, not of the batch.
__device__ __forceinline__ void stage_row_chunk(uint8_t* st, int lane, int j, uint4 v) {
    *reinterpret_cast<uint4*>(st + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
}
__device__ __forceinline__ void stage_flush(const CUtensorMap* tm, uint8_t* st, int lane, int col0, int row0) {
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
        tma_store_2d(tm, st, col0, row0);
        bulk_commit();
        bulk_wait_read<0>();     // the tile has been read: shared memory may go away with the CTA
    }
    __syncwarp();
}

#define ATT_WAIT(bar, parity, code) \
    if (!mbar_wait((bar), (parity), abort_flag, p.status, (code))) goto done

// A running maximum is only raised when the new one exceeds it by more than this (log2 units): the
// probabilities then stay below 2^8 and the accumulator in TMEM rarely needs rescaling.
constexpr float kRescaleThreshold = 8.f;
constexpr int kDkvStages = 4;   // Q/dO ring of the dK/dV kernel (64-row tiles)

// ─────────────────────────────── forward ───────────────────────────────
// Two independent softmax streams: key tiles of even index belong to warp group 0, odd ones to group 1.
// Each group (four warps, one thread per query row) has its own score buffer, P buffer, running
// (max, sum) and output accumulator, so the TMEM reads and the exponentials of one tile overlap with those
// of the next and no group ever waits for the other; the two partial outputs are merged once at the end
// (the split-KV identity O = (O0*2^(m0-M) + O1*2^(m1-M)) / (l0*2^(m0-M) + l1*2^(m1-M))).
// TMEM: S of group g at columns [128g, 128g+128), O of group g at [256 + g*HD, 256 + (g+1)*HD).

template <int HD>
__global__ void __launch_bounds__(320, 1) attn_fwd_kernel(const __grid_constant__ AttnParams p) {
    constexpr uint32_t TB = Tile<HD>::BYTES;
    constexpr int KS = 2;   // K ring (a slot is free again once its Q.K^T has completed, two tiles before it is needed)
    constexpr uint32_t PB = 32768;   // one P tile [128 queries][128 keys] BF16; two of them, alternating by key tile
    constexpr uint32_t OFF_Q = 0, OFF_K = TB, OFF_V = (1 + KS) * TB, OFF_P = (3 + KS) * TB, OFF_BAR = (3 + KS) * TB + 2 * PB;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    uint64_t *q_full = bars, *k_full = bars + 1, *k_empty = bars + 4, *v_full = bars + 7, *v_empty = bars + 9,
             *s_full = bars + 11, *s_empty = bars + 13, *p_full = bars + 15, *o_full = bars + 17;
    uint64_t* x_bar = bars + 19;   // one per TMEM lane group: the two warps that own the same rows meet here at the end
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 23);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    if (blockDim.x != 320) {   // the warp roles below assume ten warps: refuse any other launch shape
        if (threadIdx.x == 0) atomicCAS(p.status, 0, int(DS_BAD_LAUNCH));
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // 1-D grid ordered heavy-first over the WHOLE launch: late query tiles (most key tiles) of every
    // (head, batch) come before any lighter tile
    const int nt = (p.T + 127) / 128, hb = p.Hq * p.B;
    const int qt = nt - 1 - int(blockIdx.x) / hb;
    const int h = (int(blockIdx.x) % hb) % p.Hq, b = (int(blockIdx.x) % hb) / p.Hq;
    const int hk = h / (p.Hq / p.Hkv);
    const int n = qt + 1;                        // key tiles 0..qt
    const int q0 = qt * 128;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < KS; i++) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
        for (int i = 0; i < 2; i++) {
            mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4);
            mbar_init(&p_full[i], 4); mbar_init(&o_full[i], 1);
        }
        for (int i = 0; i < 4; i++) mbar_init(&x_bar[i], 2);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t TM_O = tmem + 256;

    if (warp == 0) {
        if (lane == 0) {
            mbar_arrive_expect_tx(q_full, TB);
            load_tile<HD>(smem + OFF_Q, 16384, &p.tmQ, q_full, h * HD, b * p.T + q0);
            // K and V tiles are fetched by two independent cursors: a V slot only frees when the P.V two
            // tiles back has completed, and the K tiles (needed two tiles ahead by the scores) must not queue
            // behind that wait.
            int jk = 0, jv = 0;
            uint64_t t0 = 0;
            for (uint32_t spin = 0; jk < n || jv < n; ++spin) {
                bool progress = false;
                if (jk < n && mbar_test_wait(&k_empty[jk % KS], ((jk / KS) & 1) ^ 1u)) {
                    const int kst = jk % KS;
                    mbar_arrive_expect_tx(&k_full[kst], TB);
                    load_tile<HD>(smem + OFF_K + kst * TB, 16384, &p.tmK, &k_full[kst], hk * HD, b * p.T + jk * 128);
                    jk++; progress = true;
                }
                if (jv < n && mbar_test_wait(&v_empty[jv & 1], ((jv >> 1) & 1) ^ 1u)) {
                    const int st = jv & 1;
                    mbar_arrive_expect_tx(&v_full[st], TB);
                    load_tile<HD>(smem + OFF_V + st * TB, 16384, &p.tmV, &v_full[st], hk * HD, b * p.T + jv * 128);
                    jv++; progress = true;
                }
                if (progress) { t0 = 0; continue; }
                if ((spin & 63u) == 63u) {       // bounded like every other wait of the kernel
                    if (*abort_flag) goto done;
                    const uint64_t now = globaltimer_ns();
                    if (t0 == 0) t0 = now;
                    else if (now - t0 > WAIT_LIMIT_NS) {
                        *abort_flag = 1;
                        atomicCAS(p.status, 0, int(DS_TIMEOUT_PRODUCER));
                        goto done;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint64_t dQd = desc_k(smem_u32(smem + OFF_Q)), dKd = desc_k(smem_u32(smem + OFF_K)),
                           dVd = desc_mn(smem_u32(smem + OFF_V), 16384), dPd = desc_k(smem_u32(smem + OFF_P));
            ATT_WAIT(q_full, 0, DS_TIMEOUT_MMA);
            // Two cursors, polled: the scores S(js) are issued as soon as their K tile has landed and the softmax
            // group has pulled S(js-2) into registers; O += P.V of tile jp as soon as its group has published P.
            // Neither waits behind the other - a P that is still being exponentiated must not hold back the
            // scores the OTHER group is about to need.
            int js = 0, jp = 0;
            uint64_t t0 = 0;
            for (uint32_t spin = 0; jp < n; ++spin) {
                bool progress = false;
                if (js < n) {
                    const int st = js & 1, kst = js % KS;
                    if (mbar_test_wait(&k_full[kst], (js / KS) & 1) && mbar_test_wait(&s_empty[st], ((js >> 1) & 1) ^ 1u)) {
                        tcgen05_fence_after_sync();
                        mma_kk<HD, 128>(tmem + st * 128, dQd, 16384, dKd + ((kst * TB) >> 4), 16384, false);
                        umma_commit(&k_empty[kst]);
                        umma_commit(&s_full[st]);
                        js++; progress = true;
                    }
                }
                if (jp < js) {      // O += P_j . V_j once the softmax warps have published P_j (and rescaled O)
                    const int st = jp & 1;
                    if (mbar_test_wait(&p_full[st], (jp >> 1) & 1) && mbar_test_wait(&v_full[st], (jp >> 1) & 1)) {
                        tcgen05_fence_after_sync();
                        mma_kmn<HD, 128>(TM_O + st * HD, dPd + ((st * PB) >> 4), dVd + ((st * TB) >> 4), jp > 1);
                        umma_commit(&v_empty[st]);
                        umma_commit(&o_full[st]);
                        jp++; progress = true;
                    }
                }
                if (progress) { t0 = 0; continue; }
                if ((spin & 63u) == 63u) {       // bounded like every other wait of the kernel
                    if (*abort_flag) goto done;
                    const uint64_t now = globaltimer_ns();
                    if (t0 == 0) t0 = now;
                    else if (now - t0 > WAIT_LIMIT_NS) {
                        *abort_flag = 1;
                        atomicCAS(p.status, 0, int(DS_TIMEOUT_MMA));
                        goto done;
                    }
                }
            }
        }
    } else {
        const int lg = warp & 3, grp = (warp - 2) >> 2;   // grp: 0 = even key tiles, 1 = odd key tiles
        const int row = lg * 32 + lane;
        const int q_idx = q0 + row;
        const uint32_t lane_addr = uint32_t(lg * 32) << 16;
        const uint32_t TM_OG = TM_O + grp * HD;
        float m = -INFINITY, l = 0.f;
        uint8_t* sP = smem + OFF_P + grp * PB;

        for (int j = grp; j < n; j += 2) {
            const uint32_t ph = (j >> 1) & 1;
            ATT_WAIT(&s_full[grp], ph, DS_TIMEOUT_SOFTMAX);
            tcgen05_fence_after_sync();
            const bool diag = (j == qt);
            const uint32_t ts = tmem + grp * 128 + lane_addr;
            uint32_t s[4][32];
#pragma unroll
            for (int c = 0; c < 4; c++) tmem_ld_x32(ts + c * 32, s[c]);
            tmem_ld_wait();
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[grp]);   // the scores are in registers: S buffer is free
            if (diag) {      // the diagonal tile starts at this CTA's first query, so key column > row is the future
#pragma unroll
                for (int c = 0; c < 4; c++)
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        if (c * 32 + i > row) s[c][i] = 0xff800000u;   // -inf
            }
            // row maximum of the RAW scores (the scale is positive, so it commutes with the maximum): four
            // independent chains of three-input maxima
            float mc[4];
#pragma unroll
            for (int c = 0; c < 4; c++) {
                float a = fmax3(__uint_as_float(s[c][0]), __uint_as_float(s[c][1]), __uint_as_float(s[c][2]));
#pragma unroll
                for (int i = 3; i < 31; i += 2) a = fmax3(a, __uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1]));
                mc[c] = fmaxf(a, __uint_as_float(s[c][31]));
            }
            const float mx = fmax3(mc[0], mc[1], fmaxf(mc[2], mc[3])) * p.scale_log2;
            float alpha = 1.f;
            bool rescale = false;
            if (j < 2) {
                m = mx;
            } else if (mx > m + kRescaleThreshold) {
                alpha = ex2_approx(m - mx);
                m = mx;
                rescale = true;
            }
            if (j >= 2) {
                // this group's P buffer and accumulator were last used by P.V of its previous tile (j-2), issued a
                // whole tile ago
                ATT_WAIT(&o_full[grp], ph ^ 1u, DS_TIMEOUT_SOFTMAX);
                tcgen05_fence_after_sync();
                if (__any_sync(0xffffffffu, rescale)) {
                    // rare (the running maximum rose by more than the threshold): eight columns at a time, the scores
                    // of this tile are still live in registers
#pragma unroll 1
                    for (int c = 0; c < HD / 8; c++) {
                        uint32_t r[8];
                        tmem_ld_x8(TM_OG + lane_addr + c * 8, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 8; i++) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                        tmem_st_x8(TM_OG + lane_addr + c * 8, r);
                    }
                    tmem_st_wait();
                }
            }
            // p = 2^(s*scale - m): the scale rides in the fused multiply-add, two elements per instruction; every
            // eight probabilities leave for the P tile at once
            const uint64_t sc2 = pack_f32x2(p.scale_log2, p.scale_log2), nm2 = pack_f32x2(-m, -m);
            uint64_t sum2[2] = {0ull, 0ull};
#pragma unroll
            for (int c = 0; c < 4; c++)
#pragma unroll
                for (int g = 0; g < 4; g++) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const int i = g * 8 + e * 2;
                        const float2 x = unpack_f32x2(ffma2(pack_f32x2(__uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1])), sc2, nm2));
                        const float p0 = ex2_approx(x.x), p1 = ex2_approx(x.y);
                        sum2[e & 1] = fadd2(sum2[e & 1], pack_f32x2(p0, p1));
                        w[e] = pack_bf16x2(p0, p1);
                    }
                    *reinterpret_cast<uint4*>(sP + kmajor_off(row, c * 32 + g * 8)) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            const float2 sum_lh = unpack_f32x2(fadd2(sum2[0], sum2[1]));
            l = l * alpha + (sum_lh.x + sum_lh.y);
            fence_proxy_async_smem();
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[grp]);
        }
        // last P.V of this group, then the two groups exchange (max, sum) per row through their idle P buffers
        const int cnt = (n - grp + 1) / 2;   // key tiles this group processed
        if (cnt > 0) {
            ATT_WAIT(&o_full[grp], (cnt - 1) & 1, DS_TIMEOUT_SOFTMAX);
            tcgen05_fence_after_sync();
        }
        float2* mine = reinterpret_cast<float2*>(sP);
        const float2* other = reinterpret_cast<const float2*>(smem + OFF_P + (grp ^ 1) * PB);
        mine[row] = make_float2(m, l);
        __syncwarp();
        if (lane == 0) mbar_arrive(&x_bar[lg]);
        ATT_WAIT(&x_bar[lg], 0, DS_TIMEOUT_SOFTMAX);   // both groups have seen their last P.V complete
        tcgen05_fence_after_sync();
        const float2 o = other[row];
        const bool both = n > 1;                 // with a single key tile group 1 never ran: its accumulator is undefined
        const float m0 = grp == 0 ? m : o.x, l0 = grp == 0 ? l : o.y;
        const float m1 = grp == 0 ? o.x : m, l1 = grp == 0 ? o.y : l;
        const float M = both ? fmaxf(m0, m1) : m0;
        const float w0 = ex2_approx(m0 - M), w1 = both ? ex2_approx(m1 - M) : 0.f;
        const float L = l0 * w0 + l1 * w1;
        const float f0 = w0 / L, f1 = w1 / L;
        const bool ok = q_idx < p.T;
        __nv_bfloat16* orow = p.out + (size_t(b) * p.T + q_idx) * (size_t(p.Hq) * HD) + h * HD;
        // each group normalises and stores half of the head dimension
        const bool bulk = HD == 128 && q0 + 128 <= p.T;
        uint8_t* st = sP + 4096 + lg * 4096;     // past the (max, sum) exchange area of this group's idle P buffer
#pragma unroll
        for (int c = grp * (HD / 64); c < (grp + 1) * (HD / 64); c++) {
            uint32_t r0[32], r1[32];
            tmem_ld_x32(TM_O + lane_addr + c * 32, r0);
            if (both) tmem_ld_x32(TM_O + HD + lane_addr + c * 32, r1);
            tmem_ld_wait();
            if (ok) {
#pragma unroll
                for (int g = 0; g < 4; g++) {
                    uint32_t w[4];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int e = g * 8 + i * 2;
                        float a0 = __uint_as_float(r0[e]) * f0, a1 = __uint_as_float(r0[e + 1]) * f0;
                        if (both) { a0 += __uint_as_float(r1[e]) * f1; a1 += __uint_as_float(r1[e + 1]) * f1; }
                        w[i] = pack_bf16x2(a0, a1);
                    }
                    if (bulk) stage_row_chunk(st, lane, (c - grp * (HD / 64)) * 4 + g, make_uint4(w[0], w[1], w[2], w[3]));
                    else *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
        if (bulk) stage_flush(&p.tmOut, st, lane, h * HD + grp * 64, b * p.T + q0 + lg * 32);
        if (ok && grp == 0) p.lse[(size_t(b) * p.Hq + h) * p.T + q_idx] = M * kLn2 + logf(L);
    }
done:
    __syncwarp();
    if (*abort_flag) for (int i = 0; i < 200; i++) __nanosleep(1000);
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) { tcgen05_fence_after_sync(); tmem_dealloc(tmem, 512); }
}

// delta[b,h,t] = sum_d dO[bt, h*hd+d] * O[bt, h*hd+d].  One warp per token walks the whole row with
// 16-byte loads; a head is hd/8 consecutive vectors, i.e. a group of 16 (hd=128) or 8 (hd=64) lanes.
__global__ void __launch_bounds__(256) attn_delta_kernel(const __nv_bfloat16* __restrict__ dO,
                                                         const __nv_bfloat16* __restrict__ O, float* __restrict__ delta,
                                                         int B, int T, int Hq, int hd) {
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    const int vph = hd / 8;                 // vectors per head (8 or 16)
    const int nvec = Hq * vph;
    for (long bt = blockIdx.x * long(wpb) + (threadIdx.x >> 5); bt < long(B) * T; bt += long(gridDim.x) * wpb) {
        const uint4* a = reinterpret_cast<const uint4*>(dO + bt * Hq * hd);
        const uint4* o = reinterpret_cast<const uint4*>(O + bt * Hq * hd);
        const int b = int(bt / T), t = int(bt % T);
        for (int i0 = 0; i0 < nvec; i0 += 32) {
            const int i = i0 + lane;
            float s = 0.f;
            if (i < nvec) {
                const uint4 x = a[i], y = o[i];
                const uint32_t xw[4] = {x.x, x.y, x.z, x.w}, yw[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const float2 f = unpack_bf16x2(xw[k]), g = unpack_bf16x2(yw[k]);
                    s += f.x * g.x + f.y * g.y;
                }
            }
            for (int off = vph >> 1; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
            if (i < nvec && (lane % vph) == 0) delta[(size_t(b) * Hq + i / vph) * T + t] = s;
        }
    }
}

// ─────────────────────────────── backward: dQ ───────────────────────────────
// CTA = 128 query rows of one head; keys are walked in tiles of 128, so every contraction is an N = 128 MMA (an
// N = 64 MMA re-reads the 128-row A operand for half the work and runs at shared-memory speed, ~60 clocks for
// 32).  TMEM: S[2] at columns [0,256) double buffered, dP at [256,384) single, dQ accumulator at [384, 384+HD).
// The eight element-wise warps work on ONE tile at a time, each group of four on its 64 of the 128 key columns:
//   S(j), dP(j) complete -> all warps pull their columns into registers (`loaded`) -> the MMA issuer may overwrite
//   dP with dP(j+1) -> dS = P*(dP-delta)*scale goes back, BF16 pairs, over the first 64 columns of S(j)'s buffer
//   (`ds_full`) -> dQ += dS(j).K(j) reads that A operand from tensor memory -> S(j+2) reuses the buffer (the
//   tensor pipe executes in issue order, so it cannot overwrite a dS still being read).
// While the warps work on tile j the pipe runs dP(j+1); while they work on tile j+1 it runs dQ(j) and S(j+2).

template <int HD>
__global__ void __launch_bounds__(320, 1) attn_bwd_dq_kernel(const __grid_constant__ AttnParams p) {
    constexpr uint32_t TB = Tile<HD>::BYTES;
    constexpr int KST = 3, VST = 2;   // K is held until dQ += dS.K of its tile has run, V only until dP has
    constexpr uint32_t OFF_Q = 0, OFF_DO = TB, OFF_K = 2 * TB, OFF_V = (2 + KST) * TB, OFF_BAR = (2 + KST + VST) * TB;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    uint64_t *qdo_full = bars, *k_full = bars + 1, *k_empty = bars + 4, *v_full = bars + 7, *v_empty = bars + 9,
             *s_full = bars + 11, *dp_full = bars + 13, *loaded = bars + 14, *ds_full = bars + 15, *dq_full = bars + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    if (blockDim.x != 320) {   // the warp roles below assume ten warps: refuse any other launch shape
        if (threadIdx.x == 0) atomicCAS(p.status, 0, int(DS_BAD_LAUNCH));
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nt = (p.T + 127) / 128, hb = p.Hq * p.B;
    const int qt = nt - 1 - int(blockIdx.x) / hb;   // heavy-first over the whole launch
    const int h = (int(blockIdx.x) % hb) % p.Hq, b = (int(blockIdx.x) % hb) / p.Hq;
    const int hk = h / (p.Hq / p.Hkv);
    const int n = qt + 1;          // key tiles 0 .. qt
    const int q0 = qt * 128;

    if (threadIdx.x == 0) {
        mbar_init(qdo_full, 1);
        for (int i = 0; i < KST; i++) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
        for (int i = 0; i < VST; i++) { mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
        for (int i = 0; i < 2; i++) mbar_init(&s_full[i], 1);
        mbar_init(dp_full, 1); mbar_init(loaded, 8); mbar_init(ds_full, 8); mbar_init(dq_full, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t TM_S = tmem, TM_DP = tmem + 256, TM_DQ = tmem + 384;

    if (warp == 0) {
        if (lane == 0) {
            mbar_arrive_expect_tx(qdo_full, 2 * TB);
            load_tile<HD>(smem + OFF_Q, 16384, &p.tmQ, qdo_full, h * HD, b * p.T + q0);
            load_tile<HD>(smem + OFF_DO, 16384, &p.tmdO, qdo_full, h * HD, b * p.T + q0);
            // K and V rings are filled by two independent cursors (their slots free at different times)
            int jk = 0, jv = 0;
            uint64_t t0 = 0;
            for (uint32_t spin = 0; jk < n || jv < n; ++spin) {
                bool progress = false;
                if (jk < n && mbar_test_wait(&k_empty[jk % KST], ((jk / KST) & 1) ^ 1u)) {
                    const int st = jk % KST;
                    mbar_arrive_expect_tx(&k_full[st], TB);
                    load_tile<HD>(smem + OFF_K + st * TB, 16384, &p.tmK, &k_full[st], hk * HD, b * p.T + jk * 128);
                    jk++; progress = true;
                }
                if (jv < n && mbar_test_wait(&v_empty[jv % VST], ((jv / VST) & 1) ^ 1u)) {
                    const int st = jv % VST;
                    mbar_arrive_expect_tx(&v_full[st], TB);
                    load_tile<HD>(smem + OFF_V + st * TB, 16384, &p.tmV, &v_full[st], hk * HD, b * p.T + jv * 128);
                    jv++; progress = true;
                }
                if (progress) { t0 = 0; continue; }
                if ((spin & 63u) == 63u) {       // bounded like every other wait of the kernel
                    if (*abort_flag) goto done;
                    const uint64_t now = globaltimer_ns();
                    if (t0 == 0) t0 = now;
                    else if (now - t0 > WAIT_LIMIT_NS) {
                        *abort_flag = 1;
                        atomicCAS(p.status, 0, int(DS_TIMEOUT_PRODUCER));
                        goto done;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint64_t dQd = desc_k(smem_u32(smem + OFF_Q)), dDOd = desc_k(smem_u32(smem + OFF_DO)),
                           dKk = desc_k(smem_u32(smem + OFF_K)), dVk = desc_k(smem_u32(smem + OFF_V)),
                           dKmn = desc_mn(smem_u32(smem + OFF_K), 16384);
            ATT_WAIT(qdo_full, 0, DS_TIMEOUT_MMA);
            auto scores = [&](int jn) -> bool {      // S = Q . K^T of key tile jn into buffer jn & 1
                const int ks = jn % KST;
                if (!mbar_wait(&k_full[ks], (jn / KST) & 1, abort_flag, p.status, DS_TIMEOUT_MMA)) return false;
                tcgen05_fence_after_sync();
                mma_kk<HD, 128>(TM_S + (jn & 1) * 128, dQd, 16384, dKk + ((ks * TB) >> 4), 16384, false);
                umma_commit(&s_full[jn & 1]);
                return true;
            };
            auto dprobs = [&](int jn) -> bool {      // dP = dO . V^T of key tile jn
                const int vs = jn % VST;
                if (!mbar_wait(&v_full[vs], (jn / VST) & 1, abort_flag, p.status, DS_TIMEOUT_MMA)) return false;
                tcgen05_fence_after_sync();
                mma_kk<HD, 128>(TM_DP, dDOd, 16384, dVk + ((vs * TB) >> 4), 16384, false);
                umma_commit(&v_empty[vs]);
                umma_commit(dp_full);
                return true;
            };
            if (!scores(0) || !dprobs(0)) goto done;
            if (n > 1 && !scores(1)) goto done;
            for (int j = 0; j < n; j++) {
                if (j + 1 < n) {
                    ATT_WAIT(loaded, j & 1, DS_TIMEOUT_MMA);      // dP(j) is in registers: its buffer is free
                    if (!dprobs(j + 1)) goto done;
                }
                ATT_WAIT(ds_full, j & 1, DS_TIMEOUT_MMA);         // dS of tile j is in TMEM
                tcgen05_fence_after_sync();
                mma_tmn<HD, 128>(TM_DQ, TM_S + (j & 1) * 128, dKmn + (((j % KST) * TB) >> 4), j > 0);   // dQ += dS . K
                umma_commit(&k_empty[j % KST]);
                if (j + 2 < n && !scores(j + 2)) goto done;       // reuses the buffer dS(j) was just read from
            }
            umma_commit(dq_full);
        }
    } else {
        const int lg = warp & 3, grp = (warp - 2) >> 2;   // grp: which 64 of the tile's 128 key columns
        const int row = lg * 32 + lane;
        const int q_idx = q0 + row;
        const bool ok = q_idx < p.T;
        const uint32_t lane_addr = uint32_t(lg * 32) << 16;
        const size_t stat = (size_t(b) * p.Hq + h) * p.T + q_idx;
        const float lse2 = ok ? p.lse[stat] * kLog2e : INFINITY;
        const float dlt = ok ? p.delta[stat] : 0.f;
        const uint64_t sc2 = pack_f32x2(p.scale_log2, p.scale_log2), nl2 = pack_f32x2(-lse2, -lse2);
        const uint64_t scale2 = pack_f32x2(p.scale, p.scale), nd2 = pack_f32x2(-dlt * p.scale, -dlt * p.scale);
        for (int j = 0; j < n; j++) {
            const uint32_t tS = TM_S + (j & 1) * 128 + lane_addr;
            ATT_WAIT(&s_full[j & 1], (j >> 1) & 1, DS_TIMEOUT_SOFTMAX);
            ATT_WAIT(dp_full, j & 1, DS_TIMEOUT_SOFTMAX);
            tcgen05_fence_after_sync();
            uint32_t rs[2][32], rp[2][32];
#pragma unroll
            for (int c = 0; c < 2; c++) {
                tmem_ld_x32(tS + grp * 64 + c * 32, rs[c]);
                tmem_ld_x32(TM_DP + lane_addr + grp * 64 + c * 32, rp[c]);
            }
            tmem_ld_wait();
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(loaded);
            if (j == qt) {      // the diagonal tile starts at this CTA's first query: key column > row is the future
#pragma unroll
                for (int c = 0; c < 2; c++)
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        if (grp * 64 + c * 32 + i > row) rs[c][i] = 0xff800000u;   // -inf -> probability 0
            }
            // p = 2^(s*scale*log2e - lse*log2e), dS = p * (dP - delta) * scale: two elements per instruction
            uint32_t pk[32];
#pragma unroll
            for (int c = 0; c < 2; c++)
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const float2 a = unpack_f32x2(ffma2(pack_f32x2(__uint_as_float(rs[c][i]), __uint_as_float(rs[c][i + 1])), sc2, nl2));
                    const uint64_t pp = pack_f32x2(ex2_approx(a.x), ex2_approx(a.y));
                    const uint64_t t = ffma2(pack_f32x2(__uint_as_float(rp[c][i]), __uint_as_float(rp[c][i + 1])), scale2, nd2);
                    const float2 ds = unpack_f32x2(fmul2(pp, t));
                    pk[c * 16 + (i >> 1)] = pack_bf16x2(ds.x, ds.y);
                }
            // dS goes over columns [32 grp, 32 grp + 32) of the score buffer; those hold scores of the OTHER group's
            // half when grp == 1, so every warp must have pulled its scores first
            ATT_WAIT(loaded, j & 1, DS_TIMEOUT_SOFTMAX);
            tcgen05_fence_after_sync();
            tmem_st_x32(tS + grp * 32, pk);
            tmem_st_wait();
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(ds_full);
        }
        ATT_WAIT(dq_full, 0, DS_TIMEOUT_SOFTMAX);
        tcgen05_fence_after_sync();
        __nv_bfloat16* orow = p.out + (size_t(b) * p.T + q_idx) * (size_t(p.Hq) * HD) + h * HD;
        const bool bulk = HD == 128 && q0 + 128 <= p.T;
        uint8_t* st = smem + OFF_K + (warp - 2) * 4096;     // the K ring is idle once dq_full has fired
#pragma unroll
        for (int c = grp * (HD / 64); c < (grp + 1) * (HD / 64); c++) {   // each group stores half of the head dimension
            uint32_t r[32];
            tmem_ld_x32(TM_DQ + lane_addr + c * 32, r);
            tmem_ld_wait();
            if (ok) {
#pragma unroll
                for (int g = 0; g < 4; g++) {
                    uint32_t w[4];
#pragma unroll
                    for (int i = 0; i < 4; i++)
                        w[i] = pack_bf16x2(__uint_as_float(r[g * 8 + i * 2]), __uint_as_float(r[g * 8 + i * 2 + 1]));
                    if (bulk) stage_row_chunk(st, lane, (c - grp * (HD / 64)) * 4 + g, make_uint4(w[0], w[1], w[2], w[3]));
                    else *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
        if (bulk) stage_flush(&p.tmOut, st, lane, h * HD + grp * 64, b * p.T + q0 + lg * 32);
    }
done:
    __syncwarp();
    if (*abort_flag) for (int i = 0; i < 200; i++) __nanosleep(1000);
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) { tcgen05_fence_after_sync(); tmem_dealloc(tmem, 512); }
}

// ─────────────────────────────── backward: dK, dV ───────────────────────────────
// CTA = 128 key rows of one KV head; queries are walked in sub-tiles of 64 rows over all query heads of
// the group.  TMEM: S^T[2] at [0,128), dP^T[2] at [128,256), dV at [256,256+HD), dK at [256+HD,256+2HD).
// P^T and dS^T never touch shared memory: each element-wise thread overwrites the first 32 columns of its
// S^T / dP^T row with the BF16 pairs, and dV += P^T.dO, dK += dS^T.Q read that A operand from TMEM.  The
// tensor pipe executes in issue order, so S^T of sub-tile it+2 (issued after dV/dK of sub-tile it) cannot
// overwrite a P^T that is still being read.

template <int HD>
__global__ void __launch_bounds__(320, 1) attn_bwd_dkv_kernel(const __grid_constant__ AttnParams p) {
    constexpr uint32_t TB = Tile<HD>::BYTES, TB64 = Tile<HD>::BYTES64;
    constexpr int QST = kDkvStages;   // Q/dO ring depth (a stage is released only after dV, dK consumed it)
    constexpr uint32_t OFF_K = 0, OFF_V = TB, OFF_Q = 2 * TB, OFF_DO = 2 * TB + QST * TB64, OFF_BAR = 2 * TB + 2 * QST * TB64,
                       OFF_STAT = OFF_BAR + 256;   // 8 warps x 128 floats of per-query statistics
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    uint64_t *kv_full = bars, *qdo_full = bars + 1, *qdo_empty = bars + 1 + QST, *s_full = bars + 1 + 2 * QST,
             *p_full = s_full + 2, *acc_full = s_full + 4;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 5);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    if (blockDim.x != 320) {   // the warp roles below assume ten warps: refuse any other launch shape
        if (threadIdx.x == 0) atomicCAS(p.status, 0, int(DS_BAD_LAUNCH));
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hbk = p.Hkv * p.B, hbkp = hbk * p.kv_parts;
    const int kt = int(blockIdx.x) / hbkp;   // key tile 0 has the most work: all its CTAs start first
    const int part = (int(blockIdx.x) % hbkp) % p.kv_parts, hb = (int(blockIdx.x) % hbkp) / p.kv_parts;
    const int hk = hb % p.Hkv, b = hb / p.Hkv;
    const int Gall = p.Hq / p.Hkv;
    // with few (key tile, KV head, batch) triples the launch is as long as its heaviest CTA: the group's query heads
    // are then shared out over kv_parts CTAs whose FP32 partial sums a second kernel adds up in a fixed order
    const int g_lo = part * Gall / p.kv_parts, G = (part + 1) * Gall / p.kv_parts - g_lo;
    const int h_lo = hk * Gall + g_lo;
    const int nq64 = (p.T + 63) / 64;
    const int per_head = nq64 - 2 * kt;      // query sub-tiles 2*kt .. nq64-1 can see these keys
    const int iters = G * per_head;
    const int kv0 = kt * 128;

    if (threadIdx.x == 0) {
        mbar_init(kv_full, 1); mbar_init(acc_full, 1);
        for (int i = 0; i < QST; i++) { mbar_init(&qdo_full[i], 1); mbar_init(&qdo_empty[i], 1); }
        for (int i = 0; i < 2; i++) {
            mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 4);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t TM_ST = tmem, TM_DPT = tmem + 128, TM_DV = tmem + 256, TM_DK = tmem + 256 + HD;

    if (warp == 0) {
        if (lane == 0) {
            mbar_arrive_expect_tx(kv_full, 2 * TB);
            load_tile<HD>(smem + OFF_K, 16384, &p.tmK, kv_full, hk * HD, b * p.T + kv0);
            load_tile<HD>(smem + OFF_V, 16384, &p.tmV, kv_full, hk * HD, b * p.T + kv0);
            for (int it = 0; it < iters; it++) {
                const int h = h_lo + it / per_head, qs = 2 * kt + it % per_head, st = it % QST;
                ATT_WAIT(&qdo_empty[st], ((it / QST) & 1) ^ 1u, DS_TIMEOUT_PRODUCER);
                mbar_arrive_expect_tx(&qdo_full[st], 2 * TB64);
                load_tile<HD>(smem + OFF_Q + st * TB64, 8192, &p.tmQ64, &qdo_full[st], h * HD, b * p.T + qs * 64);
                load_tile<HD>(smem + OFF_DO + st * TB64, 8192, &p.tmdO64, &qdo_full[st], h * HD, b * p.T + qs * 64);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint64_t dKd = desc_k(smem_u32(smem + OFF_K)), dVd = desc_k(smem_u32(smem + OFF_V)),
                           dQk = desc_k(smem_u32(smem + OFF_Q)), dDOk = desc_k(smem_u32(smem + OFF_DO)),
                           dQmn = desc_mn(smem_u32(smem + OFF_Q), 8192), dDOmn = desc_mn(smem_u32(smem + OFF_DO), 8192);
            ATT_WAIT(kv_full, 0, DS_TIMEOUT_MMA);
            auto scores = [&](int in) -> bool {      // S^T = K . Q^T and dP^T = V . dO^T of sub-tile `in`
                const int st = in & 1, qs_ = in % QST;
                if (!mbar_wait(&qdo_full[qs_], (in / QST) & 1, abort_flag, p.status, DS_TIMEOUT_MMA)) return false;
                tcgen05_fence_after_sync();
                mma_kk<HD, 64>(TM_ST + st * 64, dKd, 16384, dQk + ((qs_ * TB64) >> 4), 8192, false);
                mma_kk<HD, 64>(TM_DPT + st * 64, dVd, 16384, dDOk + ((qs_ * TB64) >> 4), 8192, false);
                umma_commit(&s_full[st]);
                return true;
            };
            for (int in = 0; in < 2 && in < iters; in++)
                if (!scores(in)) goto done;
            for (int it = 0; it < iters; it++) {
                const int qs_ = it % QST, st = it & 1;
                ATT_WAIT(&p_full[st], (it >> 1) & 1, DS_TIMEOUT_MMA);   // P^T, dS^T of sub-tile it are in TMEM
                tcgen05_fence_after_sync();
                mma_tmn<HD, 64>(TM_DV, TM_ST + st * 64, dDOmn + ((qs_ * TB64) >> 4), it > 0);     // dV += P^T . dO
                mma_tmn<HD, 64>(TM_DK, TM_DPT + st * 64, dQmn + ((qs_ * TB64) >> 4), it > 0);     // dK += dS^T . Q
                umma_commit(&qdo_empty[qs_]);
                if (it + 2 < iters && !scores(it + 2)) goto done;      // reuses the S^T / dP^T buffers just read
            }
            umma_commit(acc_full);
        }
    } else {
        // Two groups of four element-wise warps: group g owns the query sub-tiles of parity g with the
        // S^T / dP^T buffers of that parity; dK and dV are plain sums, so both groups feed the same
        // accumulators.  The per-query statistics (lse, delta) of a sub-tile are 64 values shared by every key
        // row: each warp keeps them two per lane and broadcasts them with shuffles.
        const int lg = warp & 3, grp = (warp - 2) >> 2;
        const int row = lg * 32 + lane;     // key row of this thread
        const int kv_idx = kv0 + row;
        const uint32_t lane_addr = uint32_t(lg * 32) << 16;
        // fetched one of the group's iterations ahead so the global-memory latency hides behind the
        // element-wise work of the current one; +inf -> probability 0 for padded queries
        auto fetch = [&](int it, float (&fl)[2], float (&fd)[2]) {
#pragma unroll
            for (int k = 0; k < 2; k++) {
                fl[k] = INFINITY; fd[k] = 0.f;
                if (it < iters) {
                    const int h = h_lo + it / per_head, q = (2 * kt + it % per_head) * 64 + k * 32 + lane;
                    if (q < p.T) {
                        const size_t si = (size_t(b) * p.Hq + h) * p.T + q;
                        fl[k] = p.lse[si] * kLog2e; fd[k] = p.delta[si];
                    }
                }
            }
        };
        float next_l[2], next_d[2];
        fetch(grp, next_l, next_d);
        float* stat = reinterpret_cast<float*>(smem + OFF_STAT) + (warp - 2) * 128;
        const uint64_t sc2 = pack_f32x2(p.scale_log2, p.scale_log2), scale2 = pack_f32x2(p.scale, p.scale);
        for (int it = grp; it < iters; it += 2) {
            const int qs = 2 * kt + it % per_head, st = grp;
            const uint32_t ph = (it >> 1) & 1;
            const float cl[2] = {next_l[0], next_l[1]}, cd[2] = {next_d[0], next_d[1]};
            fetch(it + 2, next_l, next_d);
            ATT_WAIT(&s_full[st], ph, DS_TIMEOUT_SOFTMAX);
            tcgen05_fence_after_sync();
            uint32_t rs[2][32], rp[2][32];
#pragma unroll
            for (int c = 0; c < 2; c++) {
                tmem_ld_x32(TM_ST + st * 64 + lane_addr + c * 32, rs[c]);
                tmem_ld_x32(TM_DPT + st * 64 + lane_addr + c * 32, rp[c]);
            }
            tmem_ld_wait();
            if (qs * 64 < kv0 + 127) {   // sub-tile on the diagonal: queries before this row's key cannot see it
                const int first = kv_idx - qs * 64;      // columns below this are masked
#pragma unroll
                for (int c = 0; c < 2; c++)
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        if (c * 32 + i < first) rs[c][i] = 0xff800000u;   // -inf -> probability 0
            }
            // the sub-tile's 64 (-lse*log2e) and 64 (-delta*scale) go through this warp's own slot of shared memory
            // and come back as broadcast 16-byte loads: four columns per load, already paired for the packed math
            stat[lane] = -cl[0]; stat[32 + lane] = -cl[1];
            stat[64 + lane] = -cd[0] * p.scale; stat[96 + lane] = -cd[1] * p.scale;
            __syncwarp();
            uint32_t pk[32], dk[32];
#pragma unroll
            for (int c = 0; c < 2; c++)
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    const ulonglong2 nl = *reinterpret_cast<const ulonglong2*>(stat + c * 32 + i);
                    const ulonglong2 nd = *reinterpret_cast<const ulonglong2*>(stat + 64 + c * 32 + i);
#pragma unroll
                    for (int hh = 0; hh < 2; hh++) {
                        const int e = i + hh * 2;
                        const float2 a = unpack_f32x2(ffma2(pack_f32x2(__uint_as_float(rs[c][e]), __uint_as_float(rs[c][e + 1])), sc2,
                                                            hh ? nl.y : nl.x));
                        const float p0 = ex2_approx(a.x), p1 = ex2_approx(a.y);
                        pk[c * 16 + (e >> 1)] = pack_bf16x2(p0, p1);
                        const uint64_t t = ffma2(pack_f32x2(__uint_as_float(rp[c][e]), __uint_as_float(rp[c][e + 1])), scale2,
                                                 hh ? nd.y : nd.x);
                        const float2 ds = unpack_f32x2(fmul2(pack_f32x2(p0, p1), t));
                        dk[c * 16 + (e >> 1)] = pack_bf16x2(ds.x, ds.y);
                    }
                }
            // P^T and dS^T go back into this thread's own rows of the S^T / dP^T buffers (first 32 columns)
            tmem_st_x32(TM_ST + st * 64 + lane_addr, pk);
            tmem_st_x32(TM_DPT + st * 64 + lane_addr, dk);
            tmem_st_wait();
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[st]);
        }
        ATT_WAIT(acc_full, 0, DS_TIMEOUT_SOFTMAX);
        tcgen05_fence_after_sync();
        const bool ok = kv_idx < p.T;
        const size_t ro = (size_t(b) * p.T + kv_idx) * (size_t(p.Hkv) * HD) + hk * HD;
        for (int which = grp; which <= grp; which++) {   // group 0 stores dV, group 1 stores dK
            __nv_bfloat16* orow = (which == 0 ? p.out3 : p.out2) + ro;
            const uint32_t ta = (which == 0 ? TM_DV : TM_DK) + lane_addr;
            // partial sums: [dK | dV][part][token][Hkv*hd] FP32
            float* prow = p.kv_parts > 1 ? p.part + ((size_t(which == 0 ? 1 : 0) * p.kv_parts + part) * p.B * p.T + size_t(b) * p.T + kv_idx) *
                                                        (size_t(p.Hkv) * HD) + hk * HD
                                         : nullptr;
#pragma unroll
            for (int c = 0; c < HD / 32; c++) {
                uint32_t r[32];
                tmem_ld_x32(ta + c * 32, r);
                tmem_ld_wait();
                if (ok && prow) {
#pragma unroll
                    for (int g = 0; g < 8; g++)
                        *reinterpret_cast<uint4*>(prow + c * 32 + g * 4) = make_uint4(r[g * 4], r[g * 4 + 1], r[g * 4 + 2], r[g * 4 + 3]);
                } else if (ok) {
#pragma unroll
                    for (int g = 0; g < 4; g++) {
                        uint32_t w[4];
#pragma unroll
                        for (int i = 0; i < 4; i++)
                            w[i] = pack_bf16x2(__uint_as_float(r[g * 8 + i * 2]), __uint_as_float(r[g * 8 + i * 2 + 1]));
                        *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }
done:
    __syncwarp();
    if (*abort_flag) for (int i = 0; i < 200; i++) __nanosleep(1000);
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) { tcgen05_fence_after_sync(); tmem_dealloc(tmem, 512); }
}

// dK / dV from the partial sums of a head-split dK/dV launch: parts added in index order, one rounding to BF16.
__global__ void __launch_bounds__(256) attn_dkv_reduce_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ dK,
                                                               __nv_bfloat16* __restrict__ dV, long n, int parts) {
    const long i = (blockIdx.x * long(blockDim.x) + threadIdx.x) * 4;
    if (i >= n) return;
#pragma unroll
    for (int w = 0; w < 2; w++) {
        const float* src = part + size_t(w) * parts * n + i;
        float4 a = *reinterpret_cast<const float4*>(src);
        for (int q = 1; q < parts; q++) {
            const float4 v = *reinterpret_cast<const float4*>(src + size_t(q) * n);
            a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
        }
        uint2 o = make_uint2(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w));
        *reinterpret_cast<uint2*>((w == 0 ? dK : dV) + i) = o;
    }
}

template <int HD> constexpr size_t fwd_smem() { return 5 * Tile<HD>::BYTES + 2 * 32768 + 256 + 1024; }
template <int HD> constexpr size_t dq_smem()  { return 7 * Tile<HD>::BYTES + 256 + 1024; }
template <int HD> constexpr size_t dkv_smem() { return 2 * Tile<HD>::BYTES + 2 * kDkvStages * Tile<HD>::BYTES64 + 256 + 8 * 512 + 1024; }

int make_maps(ta_ctx* ctx, AttnParams& p, const void* Q, const void* K, const void* V, const void* dO, int B, int T,
              int Hq, int Hkv, int hd) {
    const uint64_t rows = uint64_t(B) * T;
    int rc;
    if ((rc = get_tmap_bf16(ctx, Q, uint64_t(Hq) * hd, rows, uint64_t(Hq) * hd * 2, 64, 128, &p.tmQ))) return rc;
    if ((rc = get_tmap_bf16(ctx, K, uint64_t(Hkv) * hd, rows, uint64_t(Hkv) * hd * 2, 64, 128, &p.tmK))) return rc;
    if ((rc = get_tmap_bf16(ctx, V, uint64_t(Hkv) * hd, rows, uint64_t(Hkv) * hd * 2, 64, 128, &p.tmV))) return rc;
    if (dO) {
        if ((rc = get_tmap_bf16(ctx, dO, uint64_t(Hq) * hd, rows, uint64_t(Hq) * hd * 2, 64, 128, &p.tmdO))) return rc;
        if ((rc = get_tmap_bf16(ctx, dO, uint64_t(Hq) * hd, rows, uint64_t(Hq) * hd * 2, 64, 64, &p.tmdO64))) return rc;
        if ((rc = get_tmap_bf16(ctx, Q, uint64_t(Hq) * hd, rows, uint64_t(Hq) * hd * 2, 64, 64, &p.tmQ64))) return rc;
    }
    return TA_OK;
}

int check_shape(ta_ctx* ctx, int B, int T, int Hq, int Hkv, int hd) {
    if (B <= 0 || T <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0)
        return fail(ctx, TA_ERR_INVALID, "attention: bad B/T/heads (Hq must be a multiple of Hkv)");
    if (hd != 64 && hd != 128) return fail(ctx, TA_ERR_UNSUPPORTED, "attention: head_dim must be 64 or 128");
    return TA_OK;
}

template <typename K>
int set_smem(ta_ctx* ctx, K kernel, size_t bytes) {
    TA_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes)));
    return TA_OK;
}

}  // namespace
}  // namespace ta

using namespace ta;

extern "C" {

int ta_flash_attn_fwd(ta_ctx* ctx, const void* Q, const void* K, const void* V, void* out, float* lse, int B, int T,
                      int Hq, int Hkv, int head_dim, void* stream) {
    if (!ctx || !Q || !K || !V || !out || !lse) return fail(ctx, TA_ERR_INVALID, "flash_attn_fwd: null argument");
    if (int rc = check_shape(ctx, B, T, Hq, Hkv, head_dim)) return rc;
    AttnParams p{};
    if (int rc = make_maps(ctx, p, Q, K, V, nullptr, B, T, Hq, Hkv, head_dim)) return rc;
    p.out = static_cast<__nv_bfloat16*>(out); p.lse = lse;
    if (int rc = get_tmap_bf16(ctx, out, uint64_t(Hq) * head_dim, uint64_t(B) * T, uint64_t(Hq) * head_dim * 2, 64, 32, &p.tmOut)) return rc;
    p.B = B; p.T = T; p.Hq = Hq; p.Hkv = Hkv;
    p.scale = 1.f / std::sqrt(float(head_dim)); p.scale_log2 = p.scale * kLog2e; p.status = ctx->d_status;
    const dim3 grid(((T + 127) / 128) * Hq * B);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // causal: half the square, two contractions (S, P.V)
    ProfScope prof(ctx, s, PROF_ATTN_FWD, 2.0 * 2.0 * B * Hq * double(T) * T * head_dim * 0.5);
    if (head_dim == 128) {
        if (int rc = set_smem(ctx, attn_fwd_kernel<128>, fwd_smem<128>())) return rc;
        attn_fwd_kernel<128><<<grid, 320, fwd_smem<128>(), s>>>(p);
    } else {
        if (int rc = set_smem(ctx, attn_fwd_kernel<64>, fwd_smem<64>())) return rc;
        attn_fwd_kernel<64><<<grid, 320, fwd_smem<64>(), s>>>(p);
    }
    TA_LAUNCH_CHECK(ctx, "attn_fwd_kernel");
    return TA_OK;
}

int ta_flash_attn_bwd(ta_ctx* ctx, const void* dout, const void* Q, const void* K, const void* V, const void* out,
                      const float* lse, void* dQ, void* dK, void* dV, float* delta_scratch, int B, int T, int Hq, int Hkv,
                      int head_dim, void* stream) {
    if (!ctx || !dout || !Q || !K || !V || !out || !lse || !dQ || !dK || !dV)
        return fail(ctx, TA_ERR_INVALID, "flash_attn_bwd: null argument");
    if (int rc = check_shape(ctx, B, T, Hq, Hkv, head_dim)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int nt = (T + 127) / 128;
    // dK/dV launch: one CTA per (key tile, KV head, batch); when that is too few to fill the device twice over, the
    // query heads of a group are shared out over several CTAs (FP32 partials in the workspace, fixed-order reduce)
    const int ctas = nt * Hkv * B, G = Hq / Hkv;
    const int kv_parts = ctas >= 2 * ctx->sm_count ? 1 : std::min(G, (2 * ctx->sm_count + ctas - 1) / ctas);
    const size_t n_kv = size_t(B) * T * Hkv * head_dim;
    const size_t delta_bytes = delta_scratch ? 0 : ((size_t(B) * Hq * T * sizeof(float) + 255) & ~size_t(255));
    const size_t part_bytes = kv_parts > 1 ? 2 * size_t(kv_parts) * n_kv * sizeof(float) : 0;
    float* delta = delta_scratch;
    float* part = nullptr;
    if (delta_bytes + part_bytes) {
        void* ws = nullptr;
        if (int rc = get_workspace(ctx, delta_bytes + part_bytes, &ws)) return rc;
        if (!delta) delta = static_cast<float*>(ws);
        part = reinterpret_cast<float*>(static_cast<char*>(ws) + delta_bytes);
    }
    attn_delta_kernel<<<unsigned(std::min<long>((long(B) * T + 7) / 8, long(ctx->sm_count) * 16)), 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(dout), static_cast<const __nv_bfloat16*>(out), delta, B, T, Hq, head_dim);
    TA_LAUNCH_CHECK(ctx, "attn_delta_kernel");

    AttnParams p{};
    if (int rc = make_maps(ctx, p, Q, K, V, dout, B, T, Hq, Hkv, head_dim)) return rc;
    p.lse = const_cast<float*>(lse); p.delta = delta;
    p.B = B; p.T = T; p.Hq = Hq; p.Hkv = Hkv;
    p.scale = 1.f / std::sqrt(float(head_dim)); p.scale_log2 = p.scale * kLog2e; p.status = ctx->d_status;
    p.out = static_cast<__nv_bfloat16*>(dQ);
    if (int rc = get_tmap_bf16(ctx, dQ, uint64_t(Hq) * head_dim, uint64_t(B) * T, uint64_t(Hq) * head_dim * 2, 64, 32, &p.tmOut)) return rc;
    p.out2 = static_cast<__nv_bfloat16*>(dK);
    p.out3 = static_cast<__nv_bfloat16*>(dV);
    p.kv_parts = kv_parts; p.part = part;
    // algorithmic count: five contractions (S, dP, dV, dK, dQ) over half the square
    ProfScope prof(ctx, s, PROF_ATTN_BWD, 5.0 * 2.0 * B * Hq * double(T) * T * head_dim * 0.5);
    if (head_dim == 128) {
        if (int rc = set_smem(ctx, attn_bwd_dkv_kernel<128>, dkv_smem<128>())) return rc;
        attn_bwd_dkv_kernel<128><<<dim3(nt * Hkv * B * kv_parts), 320, dkv_smem<128>(), s>>>(p);
        TA_LAUNCH_CHECK(ctx, "attn_bwd_dkv_kernel");
        if (int rc = set_smem(ctx, attn_bwd_dq_kernel<128>, dq_smem<128>())) return rc;
        attn_bwd_dq_kernel<128><<<dim3(nt * Hq * B), 320, dq_smem<128>(), s>>>(p);
    } else {
        if (int rc = set_smem(ctx, attn_bwd_dkv_kernel<64>, dkv_smem<64>())) return rc;
        attn_bwd_dkv_kernel<64><<<dim3(nt * Hkv * B * kv_parts), 320, dkv_smem<64>(), s>>>(p);
        TA_LAUNCH_CHECK(ctx, "attn_bwd_dkv_kernel");
        if (int rc = set_smem(ctx, attn_bwd_dq_kernel<64>, dq_smem<64>())) return rc;
        attn_bwd_dq_kernel<64><<<dim3(nt * Hq * B), 320, dq_smem<64>(), s>>>(p);
    }
    TA_LAUNCH_CHECK(ctx, "attn_bwd_dq_kernel");
    if (kv_parts > 1) {
        attn_dkv_reduce_kernel<<<unsigned((n_kv / 4 + 255) / 256), 256, 0, s>>>(part, static_cast<__nv_bfloat16*>(dK),
                                                                                 static_cast<__nv_bfloat16*>(dV), long(n_kv), kv_parts);
        TA_LAUNCH_CHECK(ctx, "attn_dkv_reduce_kernel");
    }
    return TA_OK;
}

}  // extern "C"
