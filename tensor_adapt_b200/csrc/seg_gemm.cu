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
    // fused SwiGLU (see GemmOut::epi): `dual` tiles hold 128 gate columns and the 128 matching up columns
    CUtensorMap tmB2[kMaxSegments];   // dual: the "up" operand of each segment (up_w, or the up adapter's B)
    int k_half[kMaxSegments];         // dual rank-r segment: A columns [0,k_half) feed the gate half, [k_half,2k_half) the up half
    int dual, epi;
    int group_m, group_n;             // raster (decode_tile)
    CUtensorMap tmC;                  // BF16 output as 32 x 32 boxes (64 B swizzle) for the epilogue's bulk stores
    int c_tma;
    void* C2;                         // epi 1: up output; epi 2: d_up output
    void* C3;                         // epi 1: act output
    const __nv_bfloat16* gate_in;     // epi 2: forward gate / up activations
    const __nv_bfloat16* up_in;
};

constexpr int BM = 128;       // rows of one MMA / one TMEM accumulator
constexpr int BK = 64;
constexpr int kGemmThreads = 320;   // TMA warp, MMA warp, eight epilogue warps
constexpr int GROUP_M = 16;   // m-tiles per raster group when there are many n-tiles: a wave touches ~16 A and ~9 B panels

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
    static constexpr size_t SMEM = size_t(STAGES) * STAGE_BYTES + 1024 + 256 + 32768;   // ring, alignment slack, barriers, epilogue staging
};

struct TileCoord {
    int m0, n0, split;
};

// Tile order (what a wave of CTAs works on together decides what stays in L2): column bands of `group_n` n-tiles
// outermost (0 = one band), inside a band row groups of `group_m` m-tiles, inside a group m fastest.  A row group's A
// panel and a band's B panel are what consecutive waves re-use.
__device__ __forceinline__ TileCoord decode_tile(int tile, int m_tiles, int n_tiles, int bm, int bn, int group_m, int group_n) {
    const int per_split = m_tiles * n_tiles;
    TileCoord t;
    t.split = tile / per_split;
    int rem = tile - t.split * per_split;
    int n_first = 0, n_band = n_tiles;
    if (group_n > 0 && group_n < n_tiles) {
        const int per_band = m_tiles * group_n;
        const int band = rem / per_band;
        n_first = band * group_n;
        n_band = min(group_n, n_tiles - n_first);
        rem -= band * per_band;      // the last, narrower band keeps m_tiles * n_band tiles: rem stays in range
    }
    const int per_group = group_m * n_band;
    const int g = rem / per_group;
    const int first_m = g * group_m;
    const int gsz = min(group_m, m_tiles - first_m);
    const int in_g = rem - g * per_group;
    t.m0 = (first_m + in_g % gsz) * bm;
    t.n0 = (n_first + in_g / gsz) * bn;
    return t;
}

__device__ __forceinline__ uint4 pack8_bf16(const float (&o)[8]) {
    uint4 w;
    w.x = pack_bf16x2(o[0], o[1]); w.y = pack_bf16x2(o[2], o[3]); w.z = pack_bf16x2(o[4], o[5]); w.w = pack_bf16x2(o[6], o[7]);
    return w;
}
__device__ __forceinline__ void unpack8_bf16(const uint4& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 t = unpack_bf16x2(w[i]);
        f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
}
// ── coalesced epilogue traffic through a per-warp staging tile ───────────────
// tcgen05.ld hands every thread one ROW of the accumulator, so a direct store has 32 lanes writing 16 bytes to 32
// different lines - one line per cycle in the load/store unit, which made the epilogue four times longer than its
// bytes warrant.  Instead each warp owns a 32-row x 64-byte staging tile in shared memory (32 BF16 columns): threads
// write their row's four 16-byte pieces (XOR-swizzled by row pair: conflict-free both ways), and the warp then moves
// the tile with 4 lanes per row, 8 rows per instruction - full 32-byte sectors, a quarter of the line operations.
// Loads of row-distributed inputs (residual, the forward's gate / up) go the same way in reverse.
constexpr uint32_t kEpiStageBytes = 8 * 2 * 2048;   // eight epilogue warps, two tiles each

__device__ __forceinline__ int stage_slot(int r, int piece) { return r * 4 + (piece ^ ((r >> 1) & 3)); }

// thread `lane` has put its row's pieces at stage[stage_slot(lane, 0..3)]; writes the 32 x 32 tile to dst
__device__ __forceinline__ void stage_store_tile(const uint4* stage, int lane, __nv_bfloat16* dst, long ld, int row0, int col0,
                                                 int M, int N) {
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int r = i * 8 + (lane >> 2), pc = lane & 3;
        const int grow = row0 + r, gcol = col0 + pc * 8;
        if (grow < M && gcol < N) *reinterpret_cast<uint4*>(dst + size_t(grow) * ld + gcol) = stage[stage_slot(r, pc)];
    }
    __syncwarp();
}

// the reverse: the 32 x 32 tile of src lands in `mine[0..3]`, the four pieces of this thread's row (zeros outside)
__device__ __forceinline__ void stage_load_rows(uint4* stage, int lane, const __nv_bfloat16* src, long ld, int row0, int col0, int M,
                                                int N, uint4 (&mine)[4]) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int r = i * 8 + (lane >> 2), pc = lane & 3;
        const int grow = row0 + r, gcol = col0 + pc * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (grow < M && gcol < N) v = *reinterpret_cast<const uint4*>(src + size_t(grow) * ld + gcol);
        stage[stage_slot(r, pc)] = v;
    }
    __syncwarp();
#pragma unroll
    for (int g = 0; g < 4; g++) mine[g] = stage[stage_slot(lane, g)];
    __syncwarp();
}

// Drains columns [c_lo*CW, c_hi*CW) of one 128-row accumulator: TMEM -> registers -> alpha, bias, residual
// -> BF16 / FP32 store (or split-K partial).  `row` is the global output row of this thread's TMEM lane.
template <int CW>
__device__ __forceinline__ void epilogue_chunks(const SegGemmParams& p, uint32_t taddr, int row, bool row_ok, int n0,
                                                int split, int c_lo, int c_hi, uint4* stage, uint32_t& nchunk) {
    const int lane = threadIdx.x & 31;
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
        if constexpr (CW == 32) {
            if (!p.f32) {   // BF16 output: bias / residual / store through the staging tile (whole warp takes part)
                // two staging tiles per warp alternate, so the bulk store of the previous chunk may still be reading one
                // while this chunk fills the other; before a tile is reused its store must have finished reading it
                uint4* st = stage + (nchunk & 1u) * 128;
                nchunk++;
                if (p.c_tma) {
                    if (lane == 0) bulk_wait_read<1>();
                    __syncwarp();
                }
                uint4 res[4];
                if (p.residual) stage_load_rows(st, lane, p.residual, p.ldc, row - lane, col0, p.M, p.N, res);
#pragma unroll
                for (int g = 0; g < 4; g++) {
                    const int col = col0 + g * 8;
                    float o[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) o[i] = v[g * 8 + i] * p.alpha;
                    if (p.bias && col < p.N) {
                        float b[8];
                        unpack8_bf16(__ldg(reinterpret_cast<const uint4*>(p.bias + col)), b);
#pragma unroll
                        for (int i = 0; i < 8; i++) o[i] += b[i];
                    }
                    if (p.residual) {
                        float r8[8];
                        unpack8_bf16(res[g], r8);
#pragma unroll
                        for (int i = 0; i < 8; i++) o[i] += r8[i];
                    }
                    st[stage_slot(lane, g)] = pack8_bf16(o);
                }
                if (p.c_tma) {
                    // hand the tile to the TMA engine: the warp goes on to its next chunk while the 2 KB drain to global
                    // memory in the background (the staging layout IS the 64-byte-swizzled box layout)
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&p.tmC, st, col0, row - lane);
                        bulk_commit();
                    }
                } else {
                    stage_store_tile(st, lane, reinterpret_cast<__nv_bfloat16*>(p.C), p.ldc, row - lane, col0, p.M, p.N);
                }
                continue;
            }
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

__device__ __forceinline__ float bf16_round_f(float x) { return __bfloat162float(__float2bfloat16(x)); }

// Fused SwiGLU forward epilogue of a dual tile: accumulator columns [0,128) are gate columns n0g.., columns
// [128,256) the matching up columns.  Stores gate, up (both rounded to BF16 first, as ops::silu_mul_fwd reads them,
// src/backend/cuda/ops.cu:913-923) and act = silu(gate) * up, each through the staging tile.  Chunks of 32 gate
// columns [c_lo, c_hi).
__device__ __forceinline__ void epilogue_swiglu_fwd(const SegGemmParams& p, uint32_t taddr, int row, int n0g, int c_lo, int c_hi,
                                                    uint4* stage) {
    const int lane = threadIdx.x & 31, row0 = row - lane;
#pragma unroll 1
    for (int c = c_lo; c < c_hi; c++) {
        const int col0 = n0g + c * 32;
        if (col0 >= p.N) break;
        uint32_t rg[32], ru[32];
        tmem_ld_x32(taddr + c * 32, rg);
        tmem_ld_x32(taddr + 128 + c * 32, ru);
        tmem_ld_wait();
        uint4 pa[4];
#pragma unroll
        for (int g = 0; g < 4; g++) {
            float og[8], oa[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                og[i] = bf16_round_f(__uint_as_float(rg[g * 8 + i]) * p.alpha);
                const float ou = bf16_round_f(__uint_as_float(ru[g * 8 + i]) * p.alpha);
                oa[i] = __fdividef(og[i], 1.f + __expf(-og[i])) * ou;
            }
            stage[stage_slot(lane, g)] = pack8_bf16(og);
            pa[g] = pack8_bf16(oa);
        }
        stage_store_tile(stage, lane, reinterpret_cast<__nv_bfloat16*>(p.C), p.ldc, row0, col0, p.M, p.N);
#pragma unroll
        for (int g = 0; g < 4; g++) {
            float ou[8];
#pragma unroll
            for (int i = 0; i < 8; i++) ou[i] = __uint_as_float(ru[g * 8 + i]) * p.alpha;
            stage[stage_slot(lane, g)] = pack8_bf16(ou);
        }
        stage_store_tile(stage, lane, reinterpret_cast<__nv_bfloat16*>(p.C2), p.ldc, row0, col0, p.M, p.N);
#pragma unroll
        for (int g = 0; g < 4; g++) stage[stage_slot(lane, g)] = pa[g];
        stage_store_tile(stage, lane, reinterpret_cast<__nv_bfloat16*>(p.C3), p.ldc, row0, col0, p.M, p.N);
    }
}

// Fused SwiGLU backward epilogue: the accumulator is d_act; d_gate = d_act * up * silu'(gate), d_up = d_act * silu(gate)
// (src/backend/cuda/ops.cu:925-941) with the forward's gate / up fetched through the staging tile (coalesced).
__device__ __forceinline__ void epilogue_swiglu_bwd(const SegGemmParams& p, uint32_t taddr, int row, int n0, int c_lo, int c_hi,
                                                    uint4* stage) {
    const int lane = threadIdx.x & 31, row0 = row - lane;
#pragma unroll 1
    for (int c = c_lo; c < c_hi; c++) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;
        uint4 gq[4], uq[4];
        stage_load_rows(stage, lane, p.gate_in, p.ldc, row0, col0, p.M, p.N, gq);
        stage_load_rows(stage, lane, p.up_in, p.ldc, row0, col0, p.M, p.N, uq);
        uint32_t r[32];
        tmem_ld_x32(taddr + c * 32, r);
        tmem_ld_wait();
        uint4 pu[4];
#pragma unroll
        for (int g = 0; g < 4; g++) {
            float gt[8], up[8], dg[8], du[8];
            unpack8_bf16(gq[g], gt);
            unpack8_bf16(uq[g], up);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float d = __uint_as_float(r[g * 8 + i]) * p.alpha;
                const float sig = __fdividef(1.f, 1.f + __expf(-gt[i]));
                dg[i] = d * up[i] * (sig * (1.f + gt[i] * (1.f - sig)));
                du[i] = d * (gt[i] * sig);
            }
            stage[stage_slot(lane, g)] = pack8_bf16(dg);
            pu[g] = pack8_bf16(du);
        }
        stage_store_tile(stage, lane, reinterpret_cast<__nv_bfloat16*>(p.C), p.ldc, row0, col0, p.M, p.N);
#pragma unroll
        for (int g = 0; g < 4; g++) stage[stage_slot(lane, g)] = pu[g];
        stage_store_tile(stage, lane, reinterpret_cast<__nv_bfloat16*>(p.C2), p.ldc, row0, col0, p.M, p.N);
    }
}

// Which half (0 = gate, 1 = up) the 16-column MMA step at A column `c` of a dual rank-r segment feeds, and the byte
// offset of its B operand inside that half's shared-memory tile (whose first column is B column `up_k0` for the up half).
struct DualStep { int half; uint32_t b_off; };
__device__ __forceinline__ DualStep dual_step(int c, int k_half, int kb) {
    if (c < k_half) return DualStep{0, uint32_t(c - kb * BK) * 2u};
    const int up_k0 = max(kb * BK - k_half, 0);
    return DualStep{1, uint32_t(c - k_half - up_k0) * 2u};
}

template <int BN, int MH>
__global__ void __launch_bounds__(kGemmThreads, 1) seg_gemm_kernel(const __grid_constant__ SegGemmParams p) {
    using C = Cfg<BN, MH>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    // behind the ring: two 2 KB epilogue staging tiles per epilogue warp (warps 2..9), then the barrier block
    uint4* stage = reinterpret_cast<uint4*>(smem + C::STAGES * C::STAGE_BYTES) + ((threadIdx.x >> 5) >= 2 ? ((threadIdx.x >> 5) - 2) * 256 : 0);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES + kEpiStageBytes);
    uint64_t* empty = full + C::STAGES;
    uint64_t* tfull = empty + C::STAGES;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    uint32_t nchunk = 0;   // chunks this epilogue warp has staged so far (selects one of its two staging tiles)

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
    const int tile_n = (MH == 2 && BN == 256 && p.dual) ? 128 : BN;   // output columns (of gate) one tile covers
    const int n_tiles = (p.N + tile_n - 1) / tile_n;
    const int total = m_tiles * n_tiles * p.split_k;

    if (warp == 0) {
        if (lane == 0) {
            for (int s = 0; s < p.nseg; s++) {
                prefetch_tensormap(&p.tmA[s]);
                prefetch_tensormap(&p.tmB[s]);
                if (p.dual) prefetch_tensormap(&p.tmB2[s]);
            }
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < total; tile += gridDim.x) {
                const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, C::TILE_M, tile_n, p.group_m, p.group_n);
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
                        if constexpr (MH == 2 && BN == 256) {
                            if (p.dual) {   // two boxes {64, 128}: gate rows, then the matching up rows (K-major only)
                                tma_load_2d(sb, &p.tmB[s], &full[stage], kb * BK, tc.n0);
                                tma_load_2d(sb + 16384, &p.tmB2[s], &full[stage],
                                            p.k_half[s] ? max(kb * BK - p.k_half[s], 0) : kb * BK, tc.n0);
                                continue;
                            }
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
                const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, C::TILE_M, tile_n, p.group_m, p.group_n);
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
                        if (MH == 2 && BN == 256 && p.dual && p.k_half[s]) {
                            // rank-r segment of a dual tile: each 16-column step feeds one half (N = 128) of the tile;
                            // the first step of each half starts that half's accumulation if nothing came before
                            const uint32_t idesc_h = umma_idesc_bf16(BM, 128, false, false);
                            for (int ki = 0; ki < kinstr; ki++) {
                                const DualStep ds = dual_step(kb * BK + ki * 16, p.k_half[s], kb);
                                const uint64_t bd = smem_desc_sw128(sb + ds.half * 16384 + ds.b_off, 16, 1024);
#pragma unroll
                                for (int hh = 0; hh < MH; hh++)
                                    umma_bf16(d_tmem + hh * 256 + ds.half * 128, smem_desc_sw128(sa + hh * 16384 + ki * 32, 16, 1024),
                                              bd, idesc_h, acc);
                            }
                            umma_commit(&empty[stage]);
                            continue;
                        }
                        // descriptors: built once per k block, advanced by an add per MMA (the start-address field counts
                        // 16-byte units and cannot carry: shared-memory addresses stay below 256 KB)
                        const uint64_t bd0 = b_mn ? smem_desc_sw128(sb, 8192, 1024) : smem_desc_sw128(sb, 16, 1024);
                        const uint64_t ad0 = a_mn ? smem_desc_sw128(sa, 8192, 1024) : smem_desc_sw128(sa, 16, 1024);
                        const uint64_t b_step = b_mn ? (2048u >> 4) : (32u >> 4), a_step = a_mn ? (2048u >> 4) : (32u >> 4);
                        for (int ki = 0; ki < kinstr; ki++) {
#pragma unroll
                            for (int hh = 0; hh < MH; hh++)
                                umma_bf16(d_tmem + hh * 256, ad0 + ki * a_step + (a_mn ? 0u : uint32_t(hh) * (16384u >> 4)), bd0 + ki * b_step, idesc, acc);
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
            const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, C::TILE_M, tile_n, p.group_m, p.group_n);
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
                if constexpr (CW == 32) {
                    if (p.epi == 1) { if constexpr (MH == 2 && BN == 256) epilogue_swiglu_fwd(p, taddr, row, tc.n0, 0, 4, stage); continue; }
                    if (p.epi == 2) { epilogue_swiglu_bwd(p, taddr, row, tc.n0, c_lo, c_hi, stage); continue; }
                }
                epilogue_chunks<CW>(p, taddr, row, row_ok, tc.n0, tc.split, c_lo, c_hi, stage, nchunk);
            }
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[buf]);
        }
    }

done:
    __syncwarp();
    if (warp >= 2 && lane == 0) bulk_wait_all();   // this warp's output tiles have reached global memory
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
    static constexpr size_t SMEM = size_t(STAGES) * STAGE_BYTES + 1024 + 256 + 32768;
};

template <int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
    seg_gemm_pair_kernel(const __grid_constant__ SegGemmParams p) {
    using C = PairCfg<BN>;
    constexpr int HALF = BN / 2;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    // behind the ring: two 2 KB epilogue staging tiles per epilogue warp (warps 2..9), then the barrier block
    uint4* stage = reinterpret_cast<uint4*>(smem + C::STAGES * C::STAGE_BYTES) + ((threadIdx.x >> 5) >= 2 ? ((threadIdx.x >> 5) - 2) * 256 : 0);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES + kEpiStageBytes);
    uint64_t* empty = full + C::STAGES;
    uint64_t* tfull = empty + C::STAGES;
    uint64_t* tempty = tfull + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    uint32_t nchunk = 0;   // chunks this epilogue warp has staged so far (selects one of its two staging tiles)

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
                const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, 512, BN, p.group_m, p.group_n);
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
            const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, 512, BN, p.group_m, p.group_n);
            if (!mbar_wait(tfull, lt & 1u, abort_flag, p.status, DS_TIMEOUT_EPILOGUE)) goto done;
            tcgen05_fence_after_sync();
            const int row = tc.m0 + int(rank) * 256 + eh * BM + lg * 32 + lane;
            const uint32_t taddr = tmem_base + uint32_t(eh) * 256u + (uint32_t(lg * 32) << 16);
            epilogue_chunks<32>(p, taddr, row, row < p.M, tc.n0, 0, 0, BN / 32, stage, nchunk);
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty0);
        }
    }

done:
    __syncwarp();
    if (warp >= 2 && lane == 0) bulk_wait_all();   // this warp's output tiles have reached global memory
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
// cluster-wide broadcast load), but each CTA owns only 128 rows, so one accumulator takes BN <= 256 of its 512 tensor-memory
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
    static constexpr size_t SMEM = size_t(STAGES) * STAGE_BYTES + 1024 + 256 + 32768;
};

template <int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
    seg_gemm_pair2_kernel(const __grid_constant__ SegGemmParams p) {
    using C = Pair2Cfg<BN>;
    constexpr int HALF = BN / 2;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    // behind the ring: two 2 KB epilogue staging tiles per epilogue warp (warps 2..9), then the barrier block
    uint4* stage = reinterpret_cast<uint4*>(smem + C::STAGES * C::STAGE_BYTES) + ((threadIdx.x >> 5) >= 2 ? ((threadIdx.x >> 5) - 2) * 256 : 0);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES + kEpiStageBytes);
    uint64_t* empty = full + C::STAGES;
    uint64_t* tfull = empty + C::STAGES;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    uint32_t nchunk = 0;   // chunks this epilogue warp has staged so far (selects one of its two staging tiles)

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
    const int tile_n = p.dual ? 128 : BN;     // dual tiles: 128 gate columns + the 128 matching up columns
    const int n_tiles = (p.N + tile_n - 1) / tile_n;
    const int total = m_tiles * n_tiles;

    if (warp == 0) {
        if (lane == 0) {
            for (int s = 0; s < p.nseg; s++) {
                prefetch_tensormap(&p.tmA[s]);
                prefetch_tensormap(&p.tmB[s]);
                if (p.dual) prefetch_tensormap(&p.tmB2[s]);
            }
            uint32_t it = 0;
            for (int tile = pair; tile < total; tile += npairs) {
                const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, 256, tile_n, p.group_m, p.group_n);
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
                        if (p.dual) {
                            if (!p.k_half[s]) {
                                // main segment: this CTA supplies one half of the N = 256 operand - rank 0 the gate rows,
                                // rank 1 the matching up rows (box {64, 128} of its own tensor map)
                                tma_load_2d_pair(sb, rank ? &p.tmB2[s] : &p.tmB[s], fbar, kb * BK, tc.n0);
                            } else {
                                // rank-r segment: two N = 128 products, each CTA supplies 64 rows of both (boxes {64, 64})
                                tma_load_2d_pair(sb, &p.tmB[s], fbar, kb * BK, tc.n0 + int(rank) * 64);
                                tma_load_2d_pair(sb + 8192, &p.tmB2[s], fbar, max(kb * BK - p.k_half[s], 0), tc.n0 + int(rank) * 64);
                            }
                            continue;
                        }
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
            // One MMA covers 128 clocks of tensor work for the pair, so the issuing thread has ~128 clocks per MMA for
            // everything else: descriptors are built once (stage 0) and advanced with one 64-bit add (the start-address
            // field counts 16-byte units and never carries: shared-memory addresses stay below 256 KB).
            const uint32_t s0 = smem_u32(smem);
            const uint64_t a_d0 = smem_desc_sw128(s0, 16, 1024);
            const uint64_t bk_d0 = smem_desc_sw128(s0 + C::A_BYTES, 16, 1024), bmn_d0 = smem_desc_sw128(s0 + C::A_BYTES, 8192, 1024);
            const uint32_t empty0 = smem_u32(&empty[0]);
            uint32_t it = 0, lt = 0, stage = 0, ph = 0;
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
                    const uint64_t b_d0 = b_mn ? bmn_d0 : bk_d0;
                    const uint64_t b_step = b_mn ? (2048u >> 4) : (32u >> 4);
                    const bool dual_r = p.dual && p.k_half[s];
                    for (int kb = 0; kb < nkb; kb++, it++) {
                        if (!mbar_wait(&full[stage], ph, abort_flag, p.status, DS_TIMEOUT_MMA)) goto done;
                        tcgen05_fence_after_sync();
                        const uint64_t so = uint64_t(stage * C::STAGE_BYTES) >> 4;
                        const int krem = p.K[s] - kb * BK;
                        if (dual_r) {
                            const uint32_t sa = s0 + stage * C::STAGE_BYTES, sb = sa + C::A_BYTES;
                            const int kinstr = krem >= BK ? 4 : (krem + 15) / 16;
                            const uint32_t idesc_h = umma_idesc_bf16(256, 128, false, false);
                            for (int ki = 0; ki < kinstr; ki++) {
                                const DualStep ds = dual_step(kb * BK + ki * 16, p.k_half[s], kb);
                                umma_bf16_pair(d_tmem + ds.half * 128, smem_desc_sw128(sa + ki * 32, 16, 1024),
                                               smem_desc_sw128(sb + ds.half * 8192 + ds.b_off, 16, 1024), idesc_h, acc);
                            }
                        } else if (krem >= BK) {
                            const uint64_t ad = a_d0 + so, bd = b_d0 + so;
                            umma_bf16_pair(d_tmem, ad, bd, idesc, acc);
                            umma_bf16_pair(d_tmem, ad + 2, bd + b_step, idesc, 1u);
                            umma_bf16_pair(d_tmem, ad + 4, bd + 2 * b_step, idesc, 1u);
                            umma_bf16_pair(d_tmem, ad + 6, bd + 3 * b_step, idesc, 1u);
                            acc = 1;
                        } else {
                            const int kinstr = (krem + 15) / 16;
                            for (int ki = 0; ki < kinstr; ki++) {
                                umma_bf16_pair(d_tmem, a_d0 + so + 2 * ki, b_d0 + so + b_step * ki, idesc, acc);
                                acc = 1;
                            }
                        }
                        umma_commit_pair(empty0 + stage * 8);
                        umma_commit_pair(peer_empty0 + stage * 8);
                        if (++stage == C::STAGES) { stage = 0; ph ^= 1u; }
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
            const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, 256, tile_n, p.group_m, p.group_n);
            const uint32_t buf = lt & 1u, use = lt >> 1;
            if (!mbar_wait(&tfull[buf], use & 1u, abort_flag, p.status, DS_TIMEOUT_EPILOGUE)) goto done;
            tcgen05_fence_after_sync();
            const int row = tc.m0 + int(rank) * 128 + lg * 32 + lane;
            const uint32_t taddr = tmem_base + buf * 256u + (uint32_t(lg * 32) << 16);
            if (p.epi == 1)      epilogue_swiglu_fwd(p, taddr, row, tc.n0, eh * 2, eh * 2 + 2, stage);
            else if (p.epi == 2) epilogue_swiglu_bwd(p, taddr, row, tc.n0, c_lo, c_hi, stage);
            else                 epilogue_chunks<32>(p, taddr, row, row < p.M, tc.n0, 0, c_lo, c_hi, stage, nchunk);
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty0 + buf * 8);
        }
    }

done:
    __syncwarp();
    if (warp >= 2 && lane == 0) bulk_wait_all();   // this warp's output tiles have reached global memory
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

// ── CTA-pair kernel, 256 x BN pair tile, double-buffered accumulators, 128-wide k blocks ───────
// As the kernel above, but a ring stage holds a 128-wide k block (three stages of 64 KB instead of six of 32 KB): the
// issuing thread's barrier round (wait, two commits, loop) is paid once per EIGHT MMAs, as in the single-CTA 256-row
// kernel, instead of once per four - a pair tile leaves that thread one MMA per 128 clocks to hide it in and the MMA
// queue is shallow.
template <int BN>
struct Pair3Cfg {
    static constexpr int STAGES = 3;
    static constexpr int BK2 = 2 * BK;                              // a stage holds a 128-wide k block: 8 MMAs per barrier round
    static constexpr uint32_t A_BYTES = 128 * BK2 * 2;              // two 64-column chunks of [128 rows][128 B]
    static constexpr uint32_t B_BYTES = 128 * BK2 * 2;              // half tile, same shape (MN-major: two n chunks of [128 k][128 B])
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr size_t SMEM = size_t(STAGES) * STAGE_BYTES + 1024 + 256 + 32768;
};

template <int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
    seg_gemm_pair3_kernel(const __grid_constant__ SegGemmParams p) {
    using C = Pair3Cfg<BN>;
    constexpr int HALF = BN / 2;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    // behind the ring: two 2 KB epilogue staging tiles per epilogue warp (warps 2..9), then the barrier block
    uint4* stage = reinterpret_cast<uint4*>(smem + C::STAGES * C::STAGE_BYTES) + ((threadIdx.x >> 5) >= 2 ? ((threadIdx.x >> 5) - 2) * 256 : 0);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES + kEpiStageBytes);
    uint64_t* empty = full + C::STAGES;
    uint64_t* tfull = empty + C::STAGES;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    uint32_t nchunk = 0;   // chunks this epilogue warp has staged so far (selects one of its two staging tiles)

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
    const int tile_n = p.dual ? 128 : BN;     // dual tiles: 128 gate columns + the 128 matching up columns
    const int n_tiles = (p.N + tile_n - 1) / tile_n;
    const int total = m_tiles * n_tiles;

    if (warp == 0) {
        if (lane == 0) {
            for (int s = 0; s < p.nseg; s++) {
                prefetch_tensormap(&p.tmA[s]);
                prefetch_tensormap(&p.tmB[s]);
                if (p.dual) prefetch_tensormap(&p.tmB2[s]);
            }
            uint32_t it = 0;
            for (int tile = pair; tile < total; tile += npairs) {
                const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, 256, tile_n, p.group_m, p.group_n);
                const int m0 = tc.m0 + int(rank) * 128, nh = tc.n0 + int(rank) * HALF;
                for (int s = 0; s < p.nseg; s++) {
                    const int nkb = (p.K[s] + C::BK2 - 1) / C::BK2;
                    const bool b_mn = p.b_mn[s] != 0;
                    for (int kb = 0; kb < nkb; kb++, it++) {
                        const uint32_t stage = it % C::STAGES;
                        const uint32_t ph = (it / C::STAGES) & 1u;
                        if (!mbar_wait(&empty[stage], ph ^ 1u, abort_flag, p.status, DS_TIMEOUT_PRODUCER)) goto done;
                        uint8_t* sa = smem + stage * C::STAGE_BYTES;
                        uint8_t* sb = sa + C::A_BYTES;
                        const uint32_t fbar = map_to_cta(smem_u32(&full[stage]), 0);
                        const int k0 = kb * C::BK2;
                        // boxes that start past K are filled with zeros and still count their bytes
                        mbar_arrive_expect_tx_cluster(fbar, C::STAGE_BYTES);
                        tma_load_2d_pair(sa, &p.tmA[s], fbar, k0, m0);                    // box {64, 128}
                        tma_load_2d_pair(sa + 16384, &p.tmA[s], fbar, k0 + 64, m0);
                        if (p.dual) {
                            if (!p.k_half[s]) {
                                // main segment: this CTA supplies one half of the N = 256 operand - rank 0 the gate rows,
                                // rank 1 the matching up rows (boxes {64, 128} of its own tensor map)
                                const CUtensorMap* tb = rank ? &p.tmB2[s] : &p.tmB[s];
                                tma_load_2d_pair(sb, tb, fbar, k0, tc.n0);
                                tma_load_2d_pair(sb + 16384, tb, fbar, k0 + 64, tc.n0);
                            } else {
                                // rank-r segment, A = [h_gate | h_up]: per 64-wide half of the stage two N = 128 products,
                                // each CTA supplies 64 rows of both adapters (boxes {64, 64})
#pragma unroll
                                for (int j = 0; j < 2; j++) {
                                    const int kk = k0 + 64 * j;
                                    tma_load_2d_pair(sb + j * 16384, &p.tmB[s], fbar, kk, tc.n0 + int(rank) * 64);
                                    tma_load_2d_pair(sb + j * 16384 + 8192, &p.tmB2[s], fbar, max(kk - p.k_half[s], 0), tc.n0 + int(rank) * 64);
                                }
                            }
                            continue;
                        }
                        if (!b_mn) {
                            tma_load_2d_pair(sb, &p.tmB[s], fbar, k0, nh);                // box {64, 128}
                            tma_load_2d_pair(sb + 16384, &p.tmB[s], fbar, k0 + 64, nh);
                        } else {                                                          // box {64 n, 64 k} x 4
                            tma_load_2d_pair(sb, &p.tmB[s], fbar, nh, k0);
                            tma_load_2d_pair(sb + 8192, &p.tmB[s], fbar, nh, k0 + 64);
                            tma_load_2d_pair(sb + 16384, &p.tmB[s], fbar, nh + 64, k0);
                            tma_load_2d_pair(sb + 16384 + 8192, &p.tmB[s], fbar, nh + 64, k0 + 64);
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            const uint32_t peer_empty0 = map_to_cta(smem_u32(&empty[0]), 1), peer_tfull0 = map_to_cta(smem_u32(&tfull[0]), 1);
            // One MMA covers 128 clocks of tensor work for the pair, so the issuing thread has ~128 clocks per MMA for
            // everything else: descriptors are built once (stage 0) and advanced with one 64-bit add (the start-address
            // field counts 16-byte units and never carries: shared-memory addresses stay below 256 KB).
            const uint32_t s0 = smem_u32(smem);
            const uint64_t a_d0 = smem_desc_sw128(s0, 16, 1024);
            const uint64_t bk_d0 = smem_desc_sw128(s0 + C::A_BYTES, 16, 1024), bmn_d0 = smem_desc_sw128(s0 + C::A_BYTES, 16384, 1024);
            const uint32_t empty0 = smem_u32(&empty[0]);
            uint32_t lt = 0, stage = 0, ph = 0;
            for (int tile = pair; tile < total; tile += npairs, lt++) {
                const uint32_t buf = lt & 1u, use = lt >> 1;
                if (!mbar_wait(&tempty[buf], (use & 1u) ^ 1u, abort_flag, p.status, DS_TIMEOUT_MMA)) goto done;
                tcgen05_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * 256u;
                uint32_t acc = 0;
                for (int s = 0; s < p.nseg; s++) {
                    const int nkb = (p.K[s] + C::BK2 - 1) / C::BK2;
                    const bool b_mn = p.b_mn[s] != 0;
                    const uint32_t idesc = umma_idesc_bf16(256, BN, false, b_mn);
                    const uint64_t b_d0 = b_mn ? bmn_d0 : bk_d0;
                    // k advances by 16: K-major 32 B inside a 64-column chunk and 16 KB to the next chunk; MN-major 16 rows = 2 KB
                    const uint64_t b_step = b_mn ? (2048u >> 4) : (32u >> 4), b_half = b_mn ? (4 * 2048u >> 4) : (16384u >> 4);
                    for (int kb = 0; kb < nkb; kb++) {
                        if (!mbar_wait(&full[stage], ph, abort_flag, p.status, DS_TIMEOUT_MMA)) goto done;
                        tcgen05_fence_after_sync();
                        const uint64_t so = uint64_t(stage * C::STAGE_BYTES) >> 4;
                        const uint64_t ad = a_d0 + so, bd = b_d0 + so;
                        const int krem = p.K[s] - kb * C::BK2;
                        if (p.dual && p.k_half[s]) {
                            const uint32_t sa = s0 + stage * C::STAGE_BYTES, sb = sa + C::A_BYTES;
                            const uint32_t idesc_h = umma_idesc_bf16(256, 128, false, false);
                            for (int j = 0; j < 2; j++)
                                for (int ki = 0; ki < 4; ki++) {
                                    const int c = kb * C::BK2 + j * 64 + ki * 16;
                                    if (c >= p.K[s]) break;
                                    const DualStep ds = dual_step(c, p.k_half[s], 2 * kb + j);
                                    umma_bf16_pair(d_tmem + ds.half * 128, smem_desc_sw128(sa + j * 16384 + ki * 32, 16, 1024),
                                                   smem_desc_sw128(sb + j * 16384 + ds.half * 8192 + ds.b_off, 16, 1024), idesc_h, acc);
                                }
                        } else if (krem >= C::BK2) {
                            umma_bf16_pair(d_tmem, ad, bd, idesc, acc);
                            umma_bf16_pair(d_tmem, ad + 2, bd + b_step, idesc, 1u);
                            umma_bf16_pair(d_tmem, ad + 4, bd + 2 * b_step, idesc, 1u);
                            umma_bf16_pair(d_tmem, ad + 6, bd + 3 * b_step, idesc, 1u);
                            umma_bf16_pair(d_tmem, ad + 1024, bd + b_half, idesc, 1u);
                            umma_bf16_pair(d_tmem, ad + 1026, bd + b_half + b_step, idesc, 1u);
                            umma_bf16_pair(d_tmem, ad + 1028, bd + b_half + 2 * b_step, idesc, 1u);
                            umma_bf16_pair(d_tmem, ad + 1030, bd + b_half + 3 * b_step, idesc, 1u);
                            acc = 1;
                        } else {
                            const int kinstr = (krem + 15) / 16;
                            for (int ki = 0; ki < kinstr; ki++) {
                                umma_bf16_pair(d_tmem, ad + (ki >> 2) * 1024 + (ki & 3) * 2, bd + (ki >> 2) * b_half + (ki & 3) * b_step, idesc, acc);
                                acc = 1;
                            }
                        }
                        umma_commit_pair(empty0 + stage * 8);
                        umma_commit_pair(peer_empty0 + stage * 8);
                        if (++stage == C::STAGES) { stage = 0; ph ^= 1u; }
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
            const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, 256, tile_n, p.group_m, p.group_n);
            const uint32_t buf = lt & 1u, use = lt >> 1;
            if (!mbar_wait(&tfull[buf], use & 1u, abort_flag, p.status, DS_TIMEOUT_EPILOGUE)) goto done;
            tcgen05_fence_after_sync();
            const int row = tc.m0 + int(rank) * 128 + lg * 32 + lane;
            const uint32_t taddr = tmem_base + buf * 256u + (uint32_t(lg * 32) << 16);
            if (p.epi == 1)      epilogue_swiglu_fwd(p, taddr, row, tc.n0, eh * 2, eh * 2 + 2, stage);
            else if (p.epi == 2) epilogue_swiglu_bwd(p, taddr, row, tc.n0, c_lo, c_hi, stage);
            else                 epilogue_chunks<32>(p, taddr, row, row < p.M, tc.n0, 0, c_lo, c_hi, stage, nchunk);
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty0 + buf * 8);
        }
    }

done:
    __syncwarp();
    if (warp >= 2 && lane == 0) bulk_wait_all();   // this warp's output tiles have reached global memory
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

// How many CTA pairs of the mode-3 kernel the device keeps resident at once (0: the query failed).  The kernel hands
// tiles to pairs statically, so a launch must not hold more pairs than that: the rest would start when the first ones
// END and double the launch time.  Cached per device, written on first use from the context's one host thread.
template <int BN>
int pair3_resident_pairs(ta_ctx* ctx) {
    static int resident[64] = {};
    static bool known[64] = {};
    const int dev = ctx->device & 63;
    if (!known[dev]) {
        known[dev] = true;
        if (cudaFuncSetAttribute(seg_gemm_pair3_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 int(Pair3Cfg<BN>::SMEM)) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(unsigned(ctx->sm_count & ~1));
            cfg.blockDim = dim3(kGemmThreads);
            cfg.dynamicSmemBytes = Pair3Cfg<BN>::SMEM;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, seg_gemm_pair3_kernel<BN>, &cfg) == cudaSuccess) resident[dev] = n;
        }
        (void)cudaGetLastError();
    }
    return resident[dev];
}

template <int BN>
int launch_pair3(ta_ctx* ctx, cudaStream_t stream, const SegGemmParams& p, int total_pair_tiles) {
    const int resident = pair3_resident_pairs<BN>(ctx);
    if (resident <= 0) return fail(ctx, TA_ERR_CUDA, "seg_gemm: the CTA-pair kernel cannot be resident on this device");
    const int grid = 2 * std::min(total_pair_tiles, std::min(resident, ctx->sm_count / 2));
    seg_gemm_pair3_kernel<BN><<<grid, kGemmThreads, Pair3Cfg<BN>::SMEM, stream>>>(p);
    TA_LAUNCH_CHECK(ctx, "seg_gemm_pair3_kernel");
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

bool seg_gemm_supports_swiglu(const ta_ctx* ctx, int M) { return ctx && M >= 256; }

bool seg_gemm_swiglu_pays(ta_ctx* ctx, int M) {
    return seg_gemm_supports_swiglu(ctx, M) && ctx->gemm_pair == 0 && !ctx->gemm_force_bn && (ctx->sm_count % 2) == 0 &&
           pair3_resident_pairs<256>(ctx) >= ctx->sm_count / 2;
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
    const bool dual = out.epi == 1;
    if (out.epi < 0 || out.epi > 2) return fail(ctx, TA_ERR_INVALID, "seg_gemm: unknown epilogue");
    if (out.epi) {
        if (out.f32 || out.bias || out.residual || out.split_k > 1 || !out.C2 || (reinterpret_cast<uintptr_t>(out.C2) & 15))
            return fail(ctx, TA_ERR_INVALID, "seg_gemm: fused SwiGLU takes plain BF16 outputs (C, C2) without bias / residual / split-K");
        if (dual) {
            if (!seg_gemm_supports_swiglu(ctx, M) || !out.C3 || (reinterpret_cast<uintptr_t>(out.C3) & 15) || segs[0].k_half)
                return fail(ctx, TA_ERR_INVALID, "seg_gemm: fused gate/up needs M >= 256, an act output and a full-K first segment");
            for (int s = 0; s < nseg; s++)
                if (!segs[s].B2 || segs[s].a_mn || segs[s].b_mn || (segs[s].ldb2 % 8) || (reinterpret_cast<uintptr_t>(segs[s].B2) & 15) ||
                    (segs[s].k_half && (segs[s].k_half % 16 || segs[s].K != 2 * segs[s].k_half)))
                    return fail(ctx, TA_ERR_INVALID, "seg_gemm: fused gate/up segments are K-major pairs (B, B2); rank-r ones have K = 2 * k_half");
        } else if (!out.gate_in || !out.up_in || (reinterpret_cast<uintptr_t>(out.gate_in) & 15) || (reinterpret_cast<uintptr_t>(out.up_in) & 15)) {
            return fail(ctx, TA_ERR_INVALID, "seg_gemm: the SwiGLU backward epilogue needs the forward's gate and up");
        }
    }
    TileChoice tcfg = dual              ? TileChoice{256, 2}
                      : out.split_k > 1 ? TileChoice{pick_bn(N), 1}
                                        : pick_tile(ctx, M, N, dual ? 2 * ksum_all : ksum_all, any_a_mn);
    // The 256 x 256 CTA-pair kernel with 128-wide k blocks (mode 3) hides its epilogue behind the next main loop, which
    // pays when the contraction is short: measured against the best single-CTA tile on 16384-row problems it is
    // +4 % (N 18944, K 3584), +7-8 % (N 3584, K 3584), +4 % (N 512), +5 % (N 4608), but -2 to -5 % at K 18944, where
    // the epilogue is a small share and 74 concurrent tiles re-stream more panels than 148.  It is the library's
    // choice for short contractions when every two SMs can hold a pair at once; cta_pair -1 switches it off.
    const bool pair3_shape = out.split_k <= 1 && !any_a_mn && M >= 256 && (ctx->sm_count % 2) == 0;
    if (ctx->gemm_pair == 0 && !ctx->gemm_force_bn && pair3_shape && N >= 256 && ksum_all <= 8192 &&
        pair3_resident_pairs<256>(ctx) >= ctx->sm_count / 2)
        tcfg = TileChoice{256, 3};
    const bool auto_pair3 = tcfg.mh == 3;
    if (auto_pair3) tcfg.mh = 2;
    const int bn = tcfg.bn, tile_m = 128 * tcfg.mh;
    // CTA-pair kernel (512 x 256 tiles over two SMs): same A boxes as the 256-row kernel, half-width B boxes.
    // Opt-in (ta_ctx_set_gemm_tuning): measured 3-7 % slower than the single-CTA 256-row kernel on the 7B shapes.
    const bool use_pair2 = ctx->gemm_pair == 2 && bn == 256 && tcfg.mh == 2 && out.split_k <= 1 && M >= 256 && (ctx->sm_count % 2) == 0;
    const bool use_pair3 = pair3_shape && bn == 256 && tcfg.mh == 2 && (auto_pair3 || ctx->gemm_pair == 3);
    const bool use_pair = ctx->gemm_pair == 1 && out.epi == 0 && tcfg.mh == 2 && bn == 256 && out.split_k <= 1 && M >= 512 && (ctx->sm_count % 2) == 0;
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
        if (!g.a_mn) rc = get_tmap_bf16(ctx, g.A, uint64_t(g.K), uint64_t(M), uint64_t(g.lda) * 2, 64, uint32_t(use_pair2 || use_pair3 ? 128 : tile_m), &p.tmA[s]);
        else         rc = get_tmap_bf16(ctx, g.A, uint64_t(M), uint64_t(g.K), uint64_t(g.lda) * 2, 64, 64, &p.tmA[s]);
        if (rc) return rc;
        if (dual) {
            // gate / up operand pair: 128-row boxes (64-row ones for a rank-r segment on the CTA-pair kernel)
            const uint64_t kb_dim = g.k_half ? uint64_t(g.k_half) : uint64_t(g.K);
            const uint32_t box_rows = (g.k_half && (use_pair2 || use_pair3)) ? 64u : 128u;
            rc = get_tmap_bf16(ctx, g.B, kb_dim, uint64_t(N), uint64_t(g.ldb) * 2, 64, box_rows, &p.tmB[s]);
            if (!rc) rc = get_tmap_bf16(ctx, g.B2, kb_dim, uint64_t(N), uint64_t(g.ldb2) * 2, 64, box_rows, &p.tmB2[s]);
            p.k_half[s] = g.k_half;
        } else if (!g.b_mn) rc = get_tmap_bf16(ctx, g.B, uint64_t(g.K), uint64_t(N), uint64_t(g.ldb) * 2, 64, uint32_t(use_pair || use_pair2 || use_pair3 ? bn / 2 : bn), &p.tmB[s]);
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
    // Raster.  Measured DRAM reads per launch on 16384-row problems (ncu, B200): with 74 n-tiles (N = 18944) groups of 16
    // m-tiles are best (0.78-0.86 GB; 8: 1.25, 32: 2.0); with 16 n-tiles (N = 3584) a wave already spans all of N and
    // narrow groups re-stream fewer A panels (K = 18944: 4 -> 1.80 GB, 8 -> 2.04, 16 -> 2.14, 64 -> 4.5; speed within noise).
    // Column bands and L2 evict_first / evict_last hints on the operand loads were tried and raised traffic.
    p.group_m = ctx->gemm_group_m > 0 ? ctx->gemm_group_m : ((dual ? (N + 127) / 128 : (N + bn - 1) / bn) <= 24 ? 4 : GROUP_M);
    p.group_n = ctx->gemm_group_n;
    p.c_tma = 0;
    if (!out.f32 && out.epi == 0 && bn >= 32) {   // BF16 output leaves through bulk tensor stores of 32 x 32 boxes
        auto tmap_fn = out.no_host_state ? encode_tmap_bf16 : ta::get_tmap_bf16;
        if (int rc = tmap_fn(ctx, out.C, uint64_t(N), uint64_t(M), uint64_t(out.ldc) * 2, 32, 32, &p.tmC)) return rc;
        p.c_tma = 1;
    }
    p.dual = dual; p.epi = out.epi; p.C2 = out.C2; p.C3 = out.C3; p.gate_in = out.gate_in; p.up_in = out.up_in;

    const int m_tiles = (M + tile_m - 1) / tile_m, n_tiles = dual ? (N + 127) / 128 : (N + bn - 1) / bn;
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
    if (dual) {   // every segment produces N gate and N up columns; a rank-r segment contracts k_half per column
        ksum = 0;
        for (int s = 0; s < nseg; s++) ksum += 2.0 * (segs[s].k_half ? segs[s].k_half : segs[s].K);
    }
    ProfScope prof(out.no_host_state ? nullptr : ctx, stream, bn >= 128 ? PROF_GEMM : PROF_GEMM_SKINNY, 2.0 * M * N * ksum);
    int rc;
    if (use_pair3) {
        rc = launch_pair3<256>(ctx, stream, p, ((M + 255) / 256) * n_tiles);
    } else if (use_pair2) {
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
