// Segmented-K BF16 GEMM for sm_100a: TMA -> 128B-swizzled shared memory -> tcgen05.mma with the
// FP32 accumulator in TMEM -> tcgen05.ld epilogue (alpha, bias, residual, BF16/FP32 store).
//
// One persistent CTA per SM, 320 threads:
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocator + MMA issuer (one elected lane)
//   warps 2-9   epilogue: warp w owns TMEM lanes 32*(w%4) .. +31, i.e. 32 rows of a 128-row accumulator;
//               the two warps of a lane group split the accumulators (256-row tiles) or the columns
// The accumulator is double-buffered in TMEM (2 x BN columns) so the epilogue of tile i overlaps the
// main loop of tile i+1.  All waits are bounded (see ptx.cuh).
#include "seg_gemm.h"

#include <algorithm>
#include <cstdio>
#include <cstring>

#include "ptx.cuh"

namespace ta {

namespace {

struct alignas(64) SegGemmParams {
    CUtensorMap tmA[kMaxSegments];
    CUtensorMap tmB[kMaxSegments];
    int K[kMaxSegments];
    int a_mn[kMaxSegments];
    int b_mn[kMaxSegments];
    int nseg, M, N;
    int split_k, kb_per_split;
    void* C;
    long ldc;
    int f32, accumulate;
    float alpha;
    const __nv_bfloat16* bias;
    const __nv_bfloat16* residual;
    float* ws;
    long ws_split_stride;
    int* status;
};

constexpr int BM = 128;       // rows of one MMA / one TMEM accumulator
constexpr int BK = 64;
constexpr int kGemmThreads = 320;   // TMA warp, MMA warp, eight epilogue warps
constexpr int GROUP_M = 16;   // m-tiles per raster group: a wave touches ~16 A tiles and ~9 B tiles -> L2 reuse

constexpr uint32_t pow2_at_least(uint32_t v) { uint32_t p = 32; while (p < v) p <<= 1; return p; }

// MH = number of 128-row accumulators per CTA tile.  MH = 1: tile 128 x BN, accumulator double-buffered
// in TMEM so the epilogue overlaps the next main loop.  MH = 2: tile 256 x BN with two accumulators that
// share every B tile: a third less operand traffic per FLOP (the 128-row kernel is bound by operand
// delivery, not by the tensor pipe), at the price of a non-overlapped epilogue.
template <int BN, int MH>
struct Cfg {
    static constexpr int TILE_M = BM * MH;
    static constexpr uint32_t A_BYTES = TILE_M * BK * 2;
    static constexpr uint32_t B_BYTES = (BN < 64 ? 64 : (BN + 63) / 64 * 64) * BK * 2;
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = MH == 2 ? 3 : (BN >= 224) ? 4 : (BN == 128) ? 6 : 8;
    static constexpr uint32_t TMEM_COLS = MH == 2 ? 512 : pow2_at_least(2 * BN);
    static constexpr int NCHUNK_B = (BN + 63) / 64;
    static constexpr size_t SMEM = size_t(STAGES) * STAGE_BYTES + 1024 + 256;
};

struct TileCoord {
    int m0, n0, split;
};

__device__ __forceinline__ TileCoord decode_tile(int tile, int m_tiles, int n_tiles, int bm, int bn) {
    const int per_split = m_tiles * n_tiles;
    TileCoord t;
    t.split = tile / per_split;
    int rem = tile - t.split * per_split;
    const int per_group = GROUP_M * n_tiles;
    const int g = rem / per_group;
    const int first_m = g * GROUP_M;
    const int gsz = min(GROUP_M, m_tiles - first_m);
    const int in_g = rem - g * per_group;
    t.m0 = (first_m + in_g % gsz) * bm;
    t.n0 = (in_g / gsz) * bn;
    return t;
}

// Drains columns [c_lo*CW, c_hi*CW) of one 128-row accumulator: TMEM -> registers -> alpha, bias, residual
// -> BF16 / FP32 store (or split-K partial).  `row` is the global output row of this thread's TMEM lane.
template <int CW>
__device__ __forceinline__ void epilogue_chunks(const SegGemmParams& p, uint32_t taddr, int row, bool row_ok, int n0,
                                                int split, int c_lo, int c_hi) {
#pragma unroll 1
    for (int c = c_lo; c < c_hi; c++) {
        const int col0 = n0 + c * CW;
        if (col0 >= p.N) break;
        float v[CW];
        if constexpr (CW == 32) {
            uint32_t r[32];
            tmem_ld_x32(taddr + c * CW, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
        } else {
            uint32_t r[16];
            tmem_ld_x16(taddr + c * CW, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
        }
        if (!row_ok) continue;
#pragma unroll
        for (int g = 0; g < CW / 8; g++) {
            const int col = col0 + g * 8;
            if (col >= p.N) break;
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; i++) o[i] = v[g * 8 + i] * p.alpha;
            if (p.bias) {
                const uint4 b = __ldg(reinterpret_cast<const uint4*>(p.bias + col));
                const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float2 f = unpack_bf16x2(bw[i]);
                    o[2 * i] += f.x;
                    o[2 * i + 1] += f.y;
                }
            }
            if (p.f32) {
                float* dst = p.ws
                                 ? p.ws + size_t(split) * p.ws_split_stride + size_t(row) * p.N + col
                                 : reinterpret_cast<float*>(p.C) + size_t(row) * p.ldc + col;
                float4 lo = make_float4(o[0], o[1], o[2], o[3]);
                float4 hi = make_float4(o[4], o[5], o[6], o[7]);
                if (p.accumulate && !p.ws) {
                    const float4 a = *reinterpret_cast<const float4*>(dst);
                    const float4 b = *reinterpret_cast<const float4*>(dst + 4);
                    lo.x += a.x; lo.y += a.y; lo.z += a.z; lo.w += a.w;
                    hi.x += b.x; hi.y += b.y; hi.z += b.z; hi.w += b.w;
                }
                *reinterpret_cast<float4*>(dst) = lo;
                *reinterpret_cast<float4*>(dst + 4) = hi;
            } else {
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + size_t(row) * p.ldc + col;
                if (p.residual) {
                    const uint4 rr = *reinterpret_cast<const uint4*>(p.residual + size_t(row) * p.ldc + col);
                    const uint32_t rw[4] = {rr.x, rr.y, rr.z, rr.w};
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float2 f = unpack_bf16x2(rw[i]);
                        o[2 * i] += f.x;
                        o[2 * i + 1] += f.y;
                    }
                }
                uint4 w;
                w.x = pack_bf16x2(o[0], o[1]);
                w.y = pack_bf16x2(o[2], o[3]);
                w.z = pack_bf16x2(o[4], o[5]);
                w.w = pack_bf16x2(o[6], o[7]);
                *reinterpret_cast<uint4*>(dst) = w;
            }
        }
    }
}

template <int BN, int MH>
__global__ void __launch_bounds__(kGemmThreads, 1) seg_gemm_kernel(const __grid_constant__ SegGemmParams p) {
    using C = Cfg<BN, MH>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
    uint64_t* empty = full + C::STAGES;
    uint64_t* tfull = empty + C::STAGES;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&tfull[b], 1);
            mbar_init(&tempty[b], 8);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int m_tiles = (p.M + C::TILE_M - 1) / C::TILE_M;
    const int n_tiles = (p.N + BN - 1) / BN;
    const int total = m_tiles * n_tiles * p.split_k;

    if (warp == 0) {
        if (lane == 0) {
            for (int s = 0; s < p.nseg; s++) {
                prefetch_tensormap(&p.tmA[s]);
                prefetch_tensormap(&p.tmB[s]);
            }
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < total; tile += gridDim.x) {
                const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, C::TILE_M, BN);
                for (int s = 0; s < p.nseg; s++) {
                    const int nkb = (p.K[s] + BK - 1) / BK;
                    int kb_lo = 0, kb_hi = nkb;
                    if (p.split_k > 1) {
                        kb_lo = tc.split * p.kb_per_split;
                        kb_hi = min(nkb, kb_lo + p.kb_per_split);
                    }
                    const bool a_mn = p.a_mn[s] != 0, b_mn = p.b_mn[s] != 0;
                    const uint32_t tx = C::A_BYTES + (b_mn ? C::NCHUNK_B * 8192u : uint32_t(BN) * 128u);
                    for (int kb = kb_lo; kb < kb_hi; kb++, it++) {
                        const uint32_t stage = it % C::STAGES;
                        const uint32_t ph = (it / C::STAGES) & 1u;
                        if (!mbar_wait(&empty[stage], ph ^ 1u, abort_flag, p.status, DS_TIMEOUT_PRODUCER)) goto done;
                        uint8_t* sa = smem + stage * C::STAGE_BYTES;
                        uint8_t* sb = sa + C::A_BYTES;
                        mbar_arrive_expect_tx(&full[stage], tx);
                        if (!a_mn) {
                            tma_load_2d(sa, &p.tmA[s], &full[stage], kb * BK, tc.m0);   // box {64, 128*MH}
                        } else {                                                        // MH == 1 only (host)
                            tma_load_2d(sa, &p.tmA[s], &full[stage], tc.m0, kb * BK);
                            tma_load_2d(sa + 8192, &p.tmA[s], &full[stage], tc.m0 + 64, kb * BK);
                        }
                        if (!b_mn) {
                            tma_load_2d(sb, &p.tmB[s], &full[stage], kb * BK, tc.n0);
                        } else {
#pragma unroll
                            for (int c = 0; c < C::NCHUNK_B; c++)
                                tma_load_2d(sb + c * 8192, &p.tmB[s], &full[stage], tc.n0 + 64 * c, kb * BK);
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t it = 0, lt = 0;
            for (int tile = blockIdx.x; tile < total; tile += gridDim.x, lt++) {
                const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, C::TILE_M, BN);
                const uint32_t buf = MH == 2 ? 0u : (lt & 1u);
                const uint32_t use = MH == 2 ? lt : (lt >> 1);
                if (!mbar_wait(&tempty[buf], (use & 1u) ^ 1u, abort_flag, p.status, DS_TIMEOUT_MMA)) goto done;
                tcgen05_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (MH == 2 ? 0u : buf * BN);
                uint32_t acc = 0;
                for (int s = 0; s < p.nseg; s++) {
                    const int nkb = (p.K[s] + BK - 1) / BK;
                    int kb_lo = 0, kb_hi = nkb;
                    if (p.split_k > 1) {
                        kb_lo = tc.split * p.kb_per_split;
                        kb_hi = min(nkb, kb_lo + p.kb_per_split);
                    }
                    const bool a_mn = p.a_mn[s] != 0, b_mn = p.b_mn[s] != 0;
                    const uint32_t idesc = umma_idesc_bf16(BM, BN, a_mn, b_mn);
                    for (int kb = kb_lo; kb < kb_hi; kb++, it++) {
                        const uint32_t stage = it % C::STAGES;
                        const uint32_t ph = (it / C::STAGES) & 1u;
                        if (!mbar_wait(&full[stage], ph, abort_flag, p.status, DS_TIMEOUT_MMA)) goto done;
                        tcgen05_fence_after_sync();
                        const uint32_t sa = smem_u32(smem + stage * C::STAGE_BYTES);
                        const uint32_t sb = sa + C::A_BYTES;
                        const int krem = p.K[s] - kb * BK;
                        const int kinstr = krem >= BK ? 4 : (krem + 15) / 16;
                        for (int ki = 0; ki < kinstr; ki++) {
                            const uint64_t bd = b_mn ? smem_desc_sw128(sb + ki * 2048, 8192, 1024)
                                                     : smem_desc_sw128(sb + ki * 32, 16, 1024);
#pragma unroll
                            for (int hh = 0; hh < MH; hh++) {
                                const uint64_t ad = a_mn ? smem_desc_sw128(sa + ki * 2048, 8192, 1024)
                                                         : smem_desc_sw128(sa + hh * 16384 + ki * 32, 16, 1024);
                                umma_bf16(d_tmem + hh * 256, ad, bd, idesc, acc);
                            }
                            acc = 1;
                        }
                        umma_commit(&empty[stage]);
                    }
                }
                umma_commit(&tfull[buf]);
            }
        }
    } else {
        // Eight epilogue warps, two per TMEM lane group (a warp may only read lanes 32*(warp%4)..+31): with
        // 256-row tiles one takes each accumulator, with 128-row tiles each takes half of the columns, so
        // every scheduler has two warps to overlap TMEM reads with conversion and stores.
        const int lg = warp & 3;
        const int eh = (warp - 2) >> 2;
        uint32_t lt = 0;
        for (int tile = blockIdx.x; tile < total; tile += gridDim.x, lt++) {
            const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, C::TILE_M, BN);
            const uint32_t buf = MH == 2 ? 0u : (lt & 1u);
            const uint32_t use = MH == 2 ? lt : (lt >> 1);
            if (!mbar_wait(&tfull[buf], use & 1u, abort_flag, p.status, DS_TIMEOUT_EPILOGUE)) goto done;
            tcgen05_fence_after_sync();
            constexpr int CW = BN >= 32 ? 32 : 16;
            constexpr int NCH = BN / CW;
            const int c_lo = MH == 2 ? 0 : eh * ((NCH + 1) / 2);
            const int c_hi = MH == 2 ? NCH : (eh == 0 ? (NCH + 1) / 2 : NCH);
#pragma unroll 1
            for (int hh = (MH == 2 ? eh : 0); hh < (MH == 2 ? eh + 1 : 1); hh++) {
                const int row = tc.m0 + hh * BM + lg * 32 + lane;
                const bool row_ok = row < p.M;
                const uint32_t taddr = tmem_base + (MH == 2 ? uint32_t(hh) * 256u : buf * BN) + (uint32_t(lg * 32) << 16);
                epilogue_chunks<CW>(p, taddr, row, row_ok, tc.n0, tc.split, c_lo, c_hi);
            }
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[buf]);
        }
    }

done:
    __syncwarp();
    if (*abort_flag) {
        // give copies and MMAs already in flight time to land before shared memory / TMEM go away
        for (int i = 0; i < 200; i++) __nanosleep(1000);
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after_sync();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ── CTA-pair kernel ─────────────────────────────────────────────────────────
// Two CTAs (a cluster of two, on neighbouring SMs) work on one 512 x BN tile: each owns 256 rows (two
// accumulators, all 512 TMEM columns) and HALF of every B tile.  One thread of the rank-0 CTA issues
// tcgen05.mma.cta_group::2 instructions (M = 256: 128 rows from each CTA's shared memory, N = BN: the two
// halves of B from the two CTAs), so per FLOP each SM fills and reads a third less shared memory than the
// single-CTA 256-row kernel.  K-major A only; B K-major or MN-major; no split-K.
//
// Barriers: full[s] lives in rank 0 (both producers announce their bytes there, both CTAs' loads complete
// on it); empty[s] and tfull live in each CTA (rank 0 commits to both); tempty lives in rank 0 (the epilogue
// warps of both CTAs arrive there).  Every wait is bounded; the cluster barrier at the end keeps either
// CTA's shared memory alive until its peer is done with it.
template <int BN>
struct PairCfg {
    static constexpr int STAGES = 4;
    static constexpr uint32_t A_BYTES = 256 * BK * 2;
    static constexpr uint32_t B_BYTES = 128 * BK * 2;              // half tile (BN/2 <= 128 rows, or two 64-column chunks)
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr size_t SMEM = size_t(STAGES) * STAGE_BYTES + 1024 + 256;
};

template <int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
    seg_gemm_pair_kernel(const __grid_constant__ SegGemmParams p) {
    using C = PairCfg<BN>;
    constexpr int HALF = BN / 2;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
    uint64_t* empty = full + C::STAGES;
    uint64_t* tfull = empty + C::STAGES;
    uint64_t* tempty = tfull + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) {
            mbar_init(&full[s], 2);      // one arrive.expect_tx from each CTA's producer
            mbar_init(&empty[s], 1);
        }
        mbar_init(tfull, 1);
        mbar_init(tempty, 16);           // eight epilogue warps in each CTA
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 512);
        tmem_relinquish_pair();
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                  // the peer's barriers are initialised before anything arrives on them
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int m_tiles = (p.M + 511) / 512;
    const int n_tiles = (p.N + BN - 1) / BN;
    const int total = m_tiles * n_tiles;

    if (warp == 0) {
        if (lane == 0) {
            for (int s = 0; s < p.nseg; s++) {
                prefetch_tensormap(&p.tmA[s]);
                prefetch_tensormap(&p.tmB[s]);
            }
            uint32_t it = 0;
            for (int tile = pair; tile < total; tile += npairs) {
                const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, 512, BN);
                const int m0 = tc.m0 + int(rank) * 256, nh = tc.n0 + int(rank) * HALF;
                for (int s = 0; s < p.nseg; s++) {
                    const int nkb = (p.K[s] + BK - 1) / BK;
                    const bool b_mn = p.b_mn[s] != 0;
                    for (int kb = 0; kb < nkb; kb++, it++) {
                        const uint32_t stage = it % C::STAGES;
                        const uint32_t ph = (it / C::STAGES) & 1u;
                        if (!mbar_wait(&empty[stage], ph ^ 1u, abort_flag, p.status, DS_TIMEOUT_PRODUCER)) goto done;
                        uint8_t* sa = smem + stage * C::STAGE_BYTES;
                        uint8_t* sb = sa + C::A_BYTES;
                        const uint32_t fbar = map_to_cta(smem_u32(&full[stage]), 0);
                        mbar_arrive_expect_tx_cluster(fbar, C::STAGE_BYTES);
                        tma_load_2d_pair(sa, &p.tmA[s], fbar, kb * BK, m0);             // box {64, 256}
                        if (!b_mn) {
                            tma_load_2d_pair(sb, &p.tmB[s], fbar, kb * BK, nh);         // box {64, 128}
                        } else {
                            tma_load_2d_pair(sb, &p.tmB[s], fbar, nh, kb * BK);         // box {64, 64} x 2
                            tma_load_2d_pair(sb + 8192, &p.tmB[s], fbar, nh + 64, kb * BK);
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            const uint32_t peer_empty0 = map_to_cta(smem_u32(&empty[0]), 1), peer_tfull = map_to_cta(smem_u32(tfull), 1);
            uint32_t it = 0, lt = 0;
            for (int tile = pair; tile < total; tile += npairs, lt++) {
                if (!mbar_wait(tempty, (lt & 1u) ^ 1u, abort_flag, p.status, DS_TIMEOUT_MMA)) goto done;
                tcgen05_fence_after_sync();
                uint32_t acc = 0;
                for (int s = 0; s < p.nseg; s++) {
                    const int nkb = (p.K[s] + BK - 1) / BK;
                    const bool b_mn = p.b_mn[s] != 0;
                    const uint32_t idesc = umma_idesc_bf16(256, BN, false, b_mn);
                    for (int kb = 0; kb < nkb; kb++, it++) {
                        const uint32_t stage = it % C::STAGES;
                        const uint32_t ph = (it / C::STAGES) & 1u;
                        if (!mbar_wait(&full[stage], ph, abort_flag, p.status, DS_TIMEOUT_MMA)) goto done;
                        tcgen05_fence_after_sync();
                        const uint32_t sa = smem_u32(smem + stage * C::STAGE_BYTES);
                        const uint32_t sb = sa + C::A_BYTES;
                        const int krem = p.K[s] - kb * BK;
                        const int kinstr = krem >= BK ? 4 : (krem + 15) / 16;
                        for (int ki = 0; ki < kinstr; ki++) {
                            const uint64_t bd = b_mn ? smem_desc_sw128(sb + ki * 2048, 8192, 1024)
                                                     : smem_desc_sw128(sb + ki * 32, 16, 1024);
#pragma unroll
                            for (int hh = 0; hh < 2; hh++)
                                umma_bf16_pair(tmem_base + hh * 256, smem_desc_sw128(sa + hh * 16384 + ki * 32, 16, 1024), bd, idesc, acc);
                            acc = 1;
                        }
                        umma_commit_pair(smem_u32(&empty[stage]));
                        umma_commit_pair(peer_empty0 + stage * 8);
                    }
                }
                umma_commit_pair(smem_u32(tfull));
                umma_commit_pair(peer_tfull);
            }
        }
    } else {
        const int lg = warp & 3;
        const int eh = (warp - 2) >> 2;
        const uint32_t tempty0 = map_to_cta(smem_u32(tempty), 0);
        uint32_t lt = 0;
        for (int tile = pair; tile < total; tile += npairs, lt++) {
            const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, 512, BN);
            if (!mbar_wait(tfull, lt & 1u, abort_flag, p.status, DS_TIMEOUT_EPILOGUE)) goto done;
            tcgen05_fence_after_sync();
            const int row = tc.m0 + int(rank) * 256 + eh * BM + lg * 32 + lane;
            const uint32_t taddr = tmem_base + uint32_t(eh) * 256u + (uint32_t(lg * 32) << 16);
            epilogue_chunks<32>(p, taddr, row, row < p.M, tc.n0, 0, 0, BN / 32);
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty0);
        }
    }

done:
    __syncwarp();
    if (*abort_flag) {
        for (int i = 0; i < 200; i++) __nanosleep(1000);
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                  // neither CTA leaves while the other may still signal or read it
    if (warp == 1) {
        tcgen05_fence_after_sync();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

// ── CTA-pair kernel, 256 x BN pair tile, double-buffered accumulators ───────
// The same pairing (cluster of two, tcgen05.mma.cta_group::2 with M = 256, half of every B tile per CTA, no
// multicast load), but each CTA owns only 128 rows, so one accumulator takes BN <= 256 of its 512 tensor-memory
// columns and a second one is free: the epilogue of tile i (TMEM -> registers -> global) overlaps the main loop of
// tile i+1, which the 256-row single-CTA tiles (all 512 columns in use) cannot do.  Per FLOP a CTA fills the same
// shared memory as the 256-row kernel and the tensor core reads a third less of it.  One MMA per 16 k (the
// single-CTA 256-row kernel issues two).  K-major A only; B K-major or MN-major; no split-K.
//
// Barriers as in the kernel above: full[s] in rank 0 (count 2: one arrive.expect_tx per CTA, both CTAs' loads
// complete on it); empty[s] and tfull[b] in each CTA (rank 0 commits to both); tempty[b] in rank 0 (the epilogue
// warps of both CTAs arrive there).
template <int BN>
struct Pair2Cfg {
    static constexpr int STAGES = 6;
    static constexpr uint32_t A_BYTES = 128 * BK * 2;
    static constexpr uint32_t B_BYTES = 128 * BK * 2;              // half tile: BN/2 <= 128 rows, or two 64-column chunks
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr size_t SMEM = size_t(STAGES) * STAGE_BYTES + 1024 + 256;
};

template <int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
    seg_gemm_pair2_kernel(const __grid_constant__ SegGemmParams p) {
    using C = Pair2Cfg<BN>;
    constexpr int HALF = BN / 2;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
    uint64_t* empty = full + C::STAGES;
    uint64_t* tfull = empty + C::STAGES;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) {
            mbar_init(&full[s], 2);      // one arrive.expect_tx from each CTA's producer
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&tfull[b], 1);
            mbar_init(&tempty[b], 16);   // eight epilogue warps in each CTA
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 512);
        tmem_relinquish_pair();
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                  // the peer's barriers are initialised before anything arrives on them
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int m_tiles = (p.M + 255) / 256;
    const int n_tiles = (p.N + BN - 1) / BN;
    const int total = m_tiles * n_tiles;

    if (warp == 0) {
        if (lane == 0) {
            for (int s = 0; s < p.nseg; s++) {
                prefetch_tensormap(&p.tmA[s]);
                prefetch_tensormap(&p.tmB[s]);
            }
            uint32_t it = 0;
            for (int tile = pair; tile < total; tile += npairs) {
                const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, 256, BN);
                const int m0 = tc.m0 + int(rank) * 128, nh = tc.n0 + int(rank) * HALF;
                for (int s = 0; s < p.nseg; s++) {
                    const int nkb = (p.K[s] + BK - 1) / BK;
                    const bool b_mn = p.b_mn[s] != 0;
                    for (int kb = 0; kb < nkb; kb++, it++) {
                        const uint32_t stage = it % C::STAGES;
                        const uint32_t ph = (it / C::STAGES) & 1u;
                        if (!mbar_wait(&empty[stage], ph ^ 1u, abort_flag, p.status, DS_TIMEOUT_PRODUCER)) goto done;
                        uint8_t* sa = smem + stage * C::STAGE_BYTES;
                        uint8_t* sb = sa + C::A_BYTES;
                        const uint32_t fbar = map_to_cta(smem_u32(&full[stage]), 0);
                        mbar_arrive_expect_tx_cluster(fbar, C::STAGE_BYTES);
                        tma_load_2d_pair(sa, &p.tmA[s], fbar, kb * BK, m0);             // box {64, 128}
                        if (!b_mn) {
                            tma_load_2d_pair(sb, &p.tmB[s], fbar, kb * BK, nh);         // box {64, 128}
                        } else {
                            tma_load_2d_pair(sb, &p.tmB[s], fbar, nh, kb * BK);         // box {64, 64} x 2
                            tma_load_2d_pair(sb + 8192, &p.tmB[s], fbar, nh + 64, kb * BK);
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            const uint32_t peer_empty0 = map_to_cta(smem_u32(&empty[0]), 1), peer_tfull0 = map_to_cta(smem_u32(&tfull[0]), 1);
            uint32_t it = 0, lt = 0;
            for (int tile = pair; tile < total; tile += npairs, lt++) {
                const uint32_t buf = lt & 1u, use = lt >> 1;
                if (!mbar_wait(&tempty[buf], (use & 1u) ^ 1u, abort_flag, p.status, DS_TIMEOUT_MMA)) goto done;
                tcgen05_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * 256u;
                uint32_t acc = 0;
                for (int s = 0; s < p.nseg; s++) {
                    const int nkb = (p.K[s] + BK - 1) / BK;
                    const bool b_mn = p.b_mn[s] != 0;
                    const uint32_t idesc = umma_idesc_bf16(256, BN, false, b_mn);
                    for (int kb = 0; kb < nkb; kb++, it++) {
                        const uint32_t stage = it % C::STAGES;
                        const uint32_t ph = (it / C::STAGES) & 1u;
                        if (!mbar_wait(&full[stage], ph, abort_flag, p.status, DS_TIMEOUT_MMA)) goto done;
                        tcgen05_fence_after_sync();
                        const uint32_t sa = smem_u32(smem + stage * C::STAGE_BYTES);
                        const uint32_t sb = sa + C::A_BYTES;
                        const int krem = p.K[s] - kb * BK;
                        const int kinstr = krem >= BK ? 4 : (krem + 15) / 16;
                        for (int ki = 0; ki < kinstr; ki++) {
                            const uint64_t bd = b_mn ? smem_desc_sw128(sb + ki * 2048, 8192, 1024)
                                                     : smem_desc_sw128(sb + ki * 32, 16, 1024);
                            umma_bf16_pair(d_tmem, smem_desc_sw128(sa + ki * 32, 16, 1024), bd, idesc, acc);
                            acc = 1;
                        }
                        umma_commit_pair(smem_u32(&empty[stage]));
                        umma_commit_pair(peer_empty0 + stage * 8);
                    }
                }
                umma_commit_pair(smem_u32(&tfull[buf]));
                umma_commit_pair(peer_tfull0 + buf * 8);
            }
        }
    } else {
        // eight epilogue warps per CTA: two per TMEM lane group, each draining half of the columns
        const int lg = warp & 3;
        const int eh = (warp - 2) >> 2;
        const uint32_t tempty0 = map_to_cta(smem_u32(&tempty[0]), 0);
        constexpr int NCH = BN / 32;
        const int c_lo = eh * ((NCH + 1) / 2), c_hi = eh == 0 ? (NCH + 1) / 2 : NCH;
        uint32_t lt = 0;
        for (int tile = pair; tile < total; tile += npairs, lt++) {
            const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, 256, BN);
            const uint32_t buf = lt & 1u, use = lt >> 1;
            if (!mbar_wait(&tfull[buf], use & 1u, abort_flag, p.status, DS_TIMEOUT_EPILOGUE)) goto done;
            tcgen05_fence_after_sync();
            const int row = tc.m0 + int(rank) * 128 + lg * 32 + lane;
            const uint32_t taddr = tmem_base + buf * 256u + (uint32_t(lg * 32) << 16);
            epilogue_chunks<32>(p, taddr, row, row < p.M, tc.n0, 0, c_lo, c_hi);
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty0 + buf * 8);
        }
    }

done:
    __syncwarp();
    if (*abort_flag) {
        for (int i = 0; i < 200; i++) __nanosleep(1000);
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                  // neither CTA leaves while the other may still signal or read it
    if (warp == 1) {
        tcgen05_fence_after_sync();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

// Fixed-order reduction of split-K partials: out (+)= sum_s ws[s][m][n]; optional transposed store.
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, int splits, long split_stride, int M, int N,
                                     float* __restrict__ out, long ldo, int transpose, int accumulate) {
    const long i = blockIdx.x * long(blockDim.x) + threadIdx.x;
    if (i >= long(M) * N) return;
    // thread order follows the OUTPUT's memory order so stores coalesce
    int m, n;
    if (transpose) { n = int(i / M); m = int(i - long(n) * M); }
    else           { m = int(i / N); n = int(i - long(m) * N); }
    float s = 0.f;
    for (int k = 0; k < splits; k++) s += ws[k * split_stride + long(m) * N + n];
    float* dst = transpose ? out + long(n) * ldo + m : out + long(m) * ldo + n;
    *dst = accumulate ? *dst + s : s;
}

template <int BN, int MH>
int launch(ta_ctx* ctx, cudaStream_t stream, const SegGemmParams& p, int total_tiles) {
    static bool attr_set[64] = {};
    const int dev = ctx->device & 63;
    if (!attr_set[dev]) {
        TA_CUDA(ctx, cudaFuncSetAttribute(seg_gemm_kernel<BN, MH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          int(Cfg<BN, MH>::SMEM)));
        attr_set[dev] = true;
    }
    const int grid = std::min(total_tiles, ctx->sm_count);
    seg_gemm_kernel<BN, MH><<<grid, kGemmThreads, Cfg<BN, MH>::SMEM, stream>>>(p);
    TA_LAUNCH_CHECK(ctx, "seg_gemm_kernel");
    return TA_OK;
}

template <int BN>
int launch_pair(ta_ctx* ctx, cudaStream_t stream, const SegGemmParams& p, int total_pair_tiles) {
    static bool attr_set[64] = {};
    const int dev = ctx->device & 63;
    if (!attr_set[dev]) {
        TA_CUDA(ctx, cudaFuncSetAttribute(seg_gemm_pair_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          int(PairCfg<BN>::SMEM)));
        attr_set[dev] = true;
    }
    const int grid = 2 * std::min(total_pair_tiles, ctx->sm_count / 2);
    seg_gemm_pair_kernel<BN><<<grid, kGemmThreads, PairCfg<BN>::SMEM, stream>>>(p);
    TA_LAUNCH_CHECK(ctx, "seg_gemm_pair_kernel");
    return TA_OK;
}

template <int BN>
int launch_pair2(ta_ctx* ctx, cudaStream_t stream, const SegGemmParams& p, int total_pair_tiles) {
    static bool attr_set[64] = {};   // per-device, written on first use from the context's one host thread
    const int dev = ctx->device & 63;
    if (!attr_set[dev]) {
        TA_CUDA(ctx, cudaFuncSetAttribute(seg_gemm_pair2_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          int(Pair2Cfg<BN>::SMEM)));
        attr_set[dev] = true;
    }
    const int grid = 2 * std::min(total_pair_tiles, ctx->sm_count / 2);
    seg_gemm_pair2_kernel<BN><<<grid, kGemmThreads, Pair2Cfg<BN>::SMEM, stream>>>(p);
    TA_LAUNCH_CHECK(ctx, "seg_gemm_pair2_kernel");
    return TA_OK;
}

struct TileChoice { int bn, mh; };

// Tile shape by a small cost model: waves of tiles over the SMs x (main-loop clocks / delivery
// efficiency of the shape + non-overlapped per-tile clocks).  The efficiencies are measured ratios of
// achieved to peak tensor throughput of each shape on large problems.
TileChoice pick_tile(const ta_ctx* ctx, int M, int N, double ksum, bool any_a_mn) {
    const int sms = ctx->sm_count;
    if (N <= 16) return {16, 1};
    if (N <= 32) return {32, 1};
    if (N <= 64) return {64, 1};
    struct Cand { int bn, mh; double eff, fixed; };
    // eff = measured (tile FLOPs / 8192 per clock) / (clocks per tile) on 16384-row problems, K >= 3584
    static const Cand cands[] = {{256, 2, 0.645, 2600}, {224, 2, 0.63, 2400}, {256, 1, 0.53, 400},
                                 {224, 1, 0.50, 400},   {128, 1, 0.31, 300},  {64, 1, 0.18, 250}};
    // experiment override (ta_ctx_set_gemm_tuning), honoured where the shape allows it
    if (ctx->gemm_force_bn && (ctx->gemm_force_mh == 1 || (!any_a_mn && M >= 256)))
        return {ctx->gemm_force_bn, ctx->gemm_force_mh};
    TileChoice best{64, 1};
    double best_t = 1e300;
    for (const Cand& c : cands) {
        if (c.mh == 2 && (any_a_mn || M < 256)) continue;
        const long tiles = long((M + 128 * c.mh - 1) / (128 * c.mh)) * ((N + c.bn - 1) / c.bn);
        const long waves = (tiles + sms - 1) / sms;
        const double t = waves * (128.0 * c.mh * c.bn * ksum * 2.0 / 8192.0 / c.eff + c.fixed);
        if (t < best_t) { best_t = t; best = {c.bn, c.mh}; }
    }
    return best;
}

int pick_bn(int N) {
    if (N <= 16) return 16;
    if (N <= 32) return 32;
    if (N <= 64) return 64;
    return 128;
}

}  // namespace

int tokens_gemm_splits(const ta_ctx* ctx, int M, int N, int K) {
    const int bn = pick_bn(N);
    const int tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn);
    const int nkb = (K + BK - 1) / BK;
    // Split the token dimension so that tiles x splits fills whole waves of SMs (at most ~2 waves, at
    // least 4 k-blocks per split); >= 2 always, because the partial + fixed-order reduce path also
    // provides the += and the transposed store.
    const int sms = ctx->sm_count;
    const int smax = std::max(2, std::min({nkb / 4, 256, (2 * sms + tiles - 1) / tiles}));
    int best = 2;
    double best_u = -1;
    for (int sp = 2; sp <= smax; sp++) {
        const long ctas = long(tiles) * sp;
        const double u = double(ctas) / double((ctas + sms - 1) / sms * sms);
        if (u > best_u + 1e-9 || (u > best_u - 0.02 && sp > best && ctas <= 2L * sms)) { best_u = std::max(u, best_u); best = sp; }
    }
    return best;
}
size_t tokens_gemm_ws_bytes(const ta_ctx* ctx, int M, int N, int K) {
    return size_t(tokens_gemm_splits(ctx, M, N, K)) * M * N * sizeof(float);
}
size_t tokens_gemm_ws_bytes_max(const ta_ctx* ctx, int M, int N) {
    const int bn = pick_bn(N);
    const int tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn);
    const int smax = std::max(2, std::min(256, (2 * ctx->sm_count + tiles - 1) / tiles));
    return size_t(smax) * M * N * sizeof(float);
}

int seg_gemm(ta_ctx* ctx, cudaStream_t stream, int M, int N, const GemmSegment* segs, int nseg, const GemmOut& out) {
    if (!ctx) return TA_ERR_INVALID;
    if (nseg < 1 || nseg > kMaxSegments) return fail(ctx, TA_ERR_INVALID, "seg_gemm: 1..6 segments");
    if (M <= 0 || N <= 0 || (N % 8) != 0) return fail(ctx, TA_ERR_INVALID, "seg_gemm: M,N > 0 and N % 8 == 0 required");
    if (!out.C || (out.ldc % 8) != 0) return fail(ctx, TA_ERR_INVALID, "seg_gemm: output pointer / ldc % 8");
    if ((reinterpret_cast<uintptr_t>(out.C) & 15) || (reinterpret_cast<uintptr_t>(out.bias) & 15) ||
        (reinterpret_cast<uintptr_t>(out.residual) & 15))
        return fail(ctx, TA_ERR_INVALID, "seg_gemm: pointers must be 16-byte aligned");
    if (out.split_k > 1 && (nseg != 1 || !out.f32 || out.bias || out.residual))
        return fail(ctx, TA_ERR_INVALID, "seg_gemm: split-K needs one segment and plain fp32 output");
    if (out.transpose_out && out.split_k <= 1)
        return fail(ctx, TA_ERR_INVALID, "seg_gemm: transposed output only through the split-K reduce");
    if (out.accumulate && !out.f32) return fail(ctx, TA_ERR_INVALID, "seg_gemm: accumulate needs fp32 output");

    double ksum_all = 0;
    bool any_a_mn = false;
    for (int s = 0; s < nseg; s++) { ksum_all += segs[s].K; any_a_mn = any_a_mn || segs[s].a_mn; }
    const TileChoice tcfg = out.split_k > 1 ? TileChoice{pick_bn(N), 1} : pick_tile(ctx, M, N, ksum_all, any_a_mn);
    const int bn = tcfg.bn, tile_m = 128 * tcfg.mh;
    // CTA-pair kernel (512 x 256 tiles over two SMs): same A boxes as the 256-row kernel, half-width B boxes.
    // Opt-in (ta_ctx_set_gemm_tuning): measured 3-7 % slower than the single-CTA 256-row kernel on the 7B shapes.
    const bool use_pair2 = ctx->gemm_pair == 2 && bn == 256 && tcfg.mh == 2 && out.split_k <= 1 && M >= 256 && (ctx->sm_count % 2) == 0;
    const bool use_pair = ctx->gemm_pair == 1 && tcfg.mh == 2 && bn == 256 && out.split_k <= 1 && M >= 512 && (ctx->sm_count % 2) == 0;
    SegGemmParams p;
    std::memset(&p, 0, sizeof(p));
    for (int s = 0; s < nseg; s++) {
        const GemmSegment& g = segs[s];
        if (!g.A || !g.B || g.K <= 0 || (g.K % 8) != 0 || (g.lda % 8) != 0 || (g.ldb % 8) != 0 ||
            (reinterpret_cast<uintptr_t>(g.A) & 15) || (reinterpret_cast<uintptr_t>(g.B) & 15))
            return fail(ctx, TA_ERR_INVALID, "seg_gemm: bad segment (null, K % 8, pitch % 8 or alignment)");
        if ((g.a_mn && (M % 8)) || (!g.a_mn && false))
            return fail(ctx, TA_ERR_INVALID, "seg_gemm: MN-major A needs M % 8 == 0");
        int rc;
        auto get_tmap_bf16 = out.no_host_state ? encode_tmap_bf16 : ta::get_tmap_bf16;
        if (!g.a_mn) rc = get_tmap_bf16(ctx, g.A, uint64_t(g.K), uint64_t(M), uint64_t(g.lda) * 2, 64, uint32_t(use_pair2 ? 128 : tile_m), &p.tmA[s]);
        else         rc = get_tmap_bf16(ctx, g.A, uint64_t(M), uint64_t(g.K), uint64_t(g.lda) * 2, 64, 64, &p.tmA[s]);
        if (rc) return rc;
        if (!g.b_mn) rc = get_tmap_bf16(ctx, g.B, uint64_t(g.K), uint64_t(N), uint64_t(g.ldb) * 2, 64, uint32_t(use_pair || use_pair2 ? bn / 2 : bn), &p.tmB[s]);
        else         rc = get_tmap_bf16(ctx, g.B, uint64_t(N), uint64_t(g.K), uint64_t(g.ldb) * 2, 64, 64, &p.tmB[s]);
        if (rc) return rc;
        p.K[s] = g.K;
        p.a_mn[s] = g.a_mn;
        p.b_mn[s] = g.b_mn;
    }
    p.nseg = nseg; p.M = M; p.N = N;
    p.C = out.C; p.ldc = out.ldc; p.f32 = out.f32; p.accumulate = out.accumulate; p.alpha = out.alpha;
    p.bias = out.bias; p.residual = out.residual; p.status = ctx->d_status;
    p.split_k = 1; p.kb_per_split = 0;

    const int m_tiles = (M + tile_m - 1) / tile_m, n_tiles = (N + bn - 1) / bn;
    if (out.split_k > 1) {
        const int nkb = (segs[0].K + BK - 1) / BK;
        const int splits = std::min(out.split_k, nkb);
        p.kb_per_split = (nkb + splits - 1) / splits;
        p.split_k = (nkb + p.kb_per_split - 1) / p.kb_per_split;   // every split is non-empty
        void* ws = nullptr;
        const size_t bytes = size_t(p.split_k) * M * N * sizeof(float);
        if (out.split_ws) {
            if (out.split_ws_bytes < bytes) return fail(ctx, TA_ERR_NOMEM, "seg_gemm: split-K scratch too small");
            ws = out.split_ws;
        } else if (int rc = get_workspace(ctx, bytes, &ws)) {
            return rc;
        }
        p.ws = static_cast<float*>(ws);
        p.ws_split_stride = long(M) * N;
    }
    const int total = m_tiles * n_tiles * p.split_k;
    double ksum = 0;
    for (int s = 0; s < nseg; s++) ksum += segs[s].K;
    ProfScope prof(out.no_host_state ? nullptr : ctx, stream, bn >= 128 ? PROF_GEMM : PROF_GEMM_SKINNY, 2.0 * M * N * ksum);
    int rc;
    if (use_pair2) {
        rc = launch_pair2<256>(ctx, stream, p, ((M + 255) / 256) * n_tiles);
    } else if (use_pair) {
        rc = launch_pair<256>(ctx, stream, p, ((M + 511) / 512) * n_tiles);
    } else if (tcfg.mh == 2) {
        rc = bn == 224 ? launch<224, 2>(ctx, stream, p, total) : launch<256, 2>(ctx, stream, p, total);
    } else {
        switch (bn) {
            case 16:  rc = launch<16, 1>(ctx, stream, p, total); break;
            case 32:  rc = launch<32, 1>(ctx, stream, p, total); break;
            case 64:  rc = launch<64, 1>(ctx, stream, p, total); break;
            case 128: rc = launch<128, 1>(ctx, stream, p, total); break;
            case 224: rc = launch<224, 1>(ctx, stream, p, total); break;
            default:  rc = launch<256, 1>(ctx, stream, p, total); break;
        }
    }
    if (rc) return rc;
    if (out.split_k > 1) {
        const long n = long(M) * N;
        splitk_reduce_kernel<<<unsigned((n + 255) / 256), 256, 0, stream>>>(
            p.ws, p.split_k, p.ws_split_stride, M, N, static_cast<float*>(out.C), out.ldc, out.transpose_out,
            out.accumulate);
        TA_LAUNCH_CHECK(ctx, "splitk_reduce_kernel");
    }
    return TA_OK;
}

}  // namespace ta
