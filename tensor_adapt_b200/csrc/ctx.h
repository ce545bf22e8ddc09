// Library context: device, status word for bounded device waits, scratch workspace and the
// tensor-map cache used by the TMA-fed kernels.  Internal header (the C ABI sees `ta_ctx` opaquely).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstddef>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/tensor_adapt_b200.h"

namespace ta {

struct TmapKey {
    const void* ptr;
    uint64_t dim0, dim1, pitch_bytes;
    uint32_t box0, box1;
    bool operator==(const TmapKey& o) const {
        return ptr == o.ptr && dim0 == o.dim0 && dim1 == o.dim1 && pitch_bytes == o.pitch_bytes && box0 == o.box0 &&
               box1 == o.box1;
    }
};
struct TmapKeyHash {
    size_t operator()(const TmapKey& k) const {
        uint64_t h = reinterpret_cast<uint64_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
        h ^= (k.dim0 + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
        h ^= (k.dim1 + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
        h ^= (k.pitch_bytes + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
        h ^= ((uint64_t(k.box0) << 32 | k.box1) + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
        return static_cast<size_t>(h);
    }
};

}  // namespace ta

struct ta_ctx {
    int device = 0;
    int sm_count = 148;
    int* d_status = nullptr;        // device word written by kernels whose waits ran out
    void* ws = nullptr;             // scratch workspace (split-K partials, reduction partials)
    size_t ws_bytes = 0;
    bool ws_owned = false;
    std::string last_error;
    std::unordered_map<ta::TmapKey, CUtensorMap, ta::TmapKeyHash> tmaps;
    long launches = 0;              // kernels launched through this context (bench.py's gpu_launches)
    // GEMM tile overrides for experiments (ta_ctx_set_gemm_tuning); 0 = let the cost model choose
    int gemm_force_bn = 0, gemm_force_mh = 0;
    int gemm_group_m = 0, gemm_group_n = 0;   // raster override (0 = built-in choice)
    int gemm_pair = 0;              // 256-wide tiles: 0 = library's choice, -1 = single-CTA kernel only, 1 / 2 / 3 = that CTA-pair kernel
    // optional per-kernel-class timing with CUDA events (off by default; see ta_profile_*)
    bool profiling = false;
    struct ProfRec { int cls; double work; cudaEvent_t e0, e1; };
    std::vector<ProfRec> prof;
};

namespace ta {
enum ProfClass { PROF_GEMM = 0, PROF_GEMM_SKINNY = 1, PROF_ATTN_FWD = 2, PROF_ATTN_BWD = 3, PROF_CLASSES = 4 };
// RAII pair of events around a launch when profiling is on; `work` is FLOPs of the launch.
struct ProfScope {
    ta_ctx* ctx; cudaStream_t s; size_t idx = size_t(-1);
    ProfScope(ta_ctx* c, cudaStream_t st, int cls, double work) : ctx(c), s(st) {
        if (!c || !c->profiling || c->prof.size() >= 200000) return;
        ta_ctx::ProfRec r{cls, work, nullptr, nullptr};
        if (cudaEventCreate(&r.e0) != cudaSuccess || cudaEventCreate(&r.e1) != cudaSuccess) return;
        cudaEventRecord(r.e0, st);
        idx = c->prof.size();
        c->prof.push_back(r);
    }
    ~ProfScope() { if (idx != size_t(-1)) cudaEventRecord(ctx->prof[idx].e1, s); }
};
}  // namespace ta

namespace ta {

int fail(ta_ctx* ctx, int code, const std::string& msg);
int check_cuda(ta_ctx* ctx, cudaError_t e, const char* what);

// Cached 2-D BF16 tensor map: tensor [dim1 rows][dim0 cols], row pitch in bytes, box [box1 rows][box0 cols], swizzle
// matching the box's inner extent (128 B for 64 columns, 64 B for 32); out-of-bounds elements read as zero and are not
// written by stores.
int get_tmap_bf16(ta_ctx* ctx, const void* ptr, uint64_t dim0, uint64_t dim1, uint64_t pitch_bytes, uint32_t box0,
                  uint32_t box1, CUtensorMap* out);

// Same map, encoded straight into *out without touching the cache (no host allocation).
int encode_tmap_bf16(ta_ctx* ctx, const void* ptr, uint64_t dim0, uint64_t dim1, uint64_t pitch_bytes, uint32_t box0,
                     uint32_t box1, CUtensorMap* out);

// Scratch of at least `bytes`, grown on demand when the context owns its workspace.
int get_workspace(ta_ctx* ctx, size_t bytes, void** out);

// Device allocation freed on scope exit (host-side helpers that return early on errors).
struct DeviceBuffer {
    void* p = nullptr;
    DeviceBuffer() = default;
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    ~DeviceBuffer() { if (p) cudaFree(p); }
    cudaError_t alloc(size_t bytes) { return cudaMalloc(&p, bytes ? bytes : 1); }
    template <typename T> T* as() const { return static_cast<T*>(p); }
};

}  // namespace ta

#define TA_CUDA(ctx, call)                                              \
    do {                                                                \
        cudaError_t _e = (call);                                        \
        if (_e != cudaSuccess) return ta::check_cuda((ctx), _e, #call); \
    } while (0)

#define TA_LAUNCH_CHECK(ctx, name)                                      \
    do {                                                                \
        cudaError_t _e = cudaGetLastError();                            \
        if (_e != cudaSuccess) return ta::check_cuda((ctx), _e, name);  \
        if (ctx) (ctx)->launches++;                                     \
    } while (0)
