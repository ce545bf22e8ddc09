// Context life-cycle, error reporting, workspace and tensor-map cache.
#include "ctx.h"

#include <cstdio>
#include <new>

namespace ta {

int fail(ta_ctx* ctx, int code, const std::string& msg) {
    if (ctx) ctx->last_error = msg;
    return code;
}

int check_cuda(ta_ctx* ctx, cudaError_t e, const char* what) {
    if (e == cudaSuccess) return TA_OK;
    return fail(ctx, TA_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

int encode_tmap_bf16(ta_ctx* ctx, const void* ptr, uint64_t dim0, uint64_t dim1, uint64_t pitch_bytes, uint32_t box0,
                     uint32_t box1, CUtensorMap* out) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(ctx, TA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (pitch_bytes & 15))
        return fail(ctx, TA_ERR_INVALID, "tensor map: base and row pitch must be multiples of 16 bytes");
    cuuint64_t gdim[2] = {dim0, dim1};
    cuuint64_t gstride[1] = {pitch_bytes};
    cuuint32_t box[2] = {box0, box1};
    cuuint32_t estr[2] = {1, 1};
    // swizzle = the inner extent of the box: 64 elements (128 B) for the MMA operand tiles, 32 elements (64 B) for the
    // 32 x 32 output tiles the GEMM epilogue stores
    const CUtensorMapSwizzle swz = box0 >= 64 ? CU_TENSOR_MAP_SWIZZLE_128B : box0 == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE;
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char buf[200];
        std::snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled failed (%d) dims=%llu x %llu pitch=%llu box=%u x %u",
                      int(r), (unsigned long long)dim0, (unsigned long long)dim1, (unsigned long long)pitch_bytes, box0,
                      box1);
        return fail(ctx, TA_ERR_CUDA, buf);
    }
    return TA_OK;
}

int get_tmap_bf16(ta_ctx* ctx, const void* ptr, uint64_t dim0, uint64_t dim1, uint64_t pitch_bytes, uint32_t box0,
                  uint32_t box1, CUtensorMap* out) {
    TmapKey key{ptr, dim0, dim1, pitch_bytes, box0, box1};
    auto it = ctx->tmaps.find(key);
    if (it != ctx->tmaps.end()) {
        *out = it->second;
        return TA_OK;
    }
    CUtensorMap m;
    if (int rc = encode_tmap_bf16(ctx, ptr, dim0, dim1, pitch_bytes, box0, box1, &m)) return rc;
    if (ctx->tmaps.size() > 8192) ctx->tmaps.clear();
    ctx->tmaps.emplace(key, m);
    *out = m;
    return TA_OK;
}

int get_workspace(ta_ctx* ctx, size_t bytes, void** out) {
    if (bytes <= ctx->ws_bytes) {
        *out = ctx->ws;
        return TA_OK;
    }
    if (!ctx->ws_owned && ctx->ws)
        return fail(ctx, TA_ERR_NOMEM, "caller-provided workspace is too small for this call");
    // growing frees the old block: drain work that may still read it
    TA_CUDA(ctx, cudaDeviceSynchronize());
    if (ctx->ws) cudaFree(ctx->ws);
    ctx->ws = nullptr;
    ctx->ws_bytes = 0;
    size_t want = bytes + (bytes >> 2) + (1u << 20);
    TA_CUDA(ctx, cudaMalloc(&ctx->ws, want));
    ctx->ws_bytes = want;
    ctx->ws_owned = true;
    *out = ctx->ws;
    return TA_OK;
}

}  // namespace ta

extern "C" {

int ta_ctx_create(int device, ta_ctx** out) {
    if (!out) return TA_ERR_INVALID;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) return TA_ERR_CUDA;
    if (cudaSetDevice(device) != cudaSuccess) return TA_ERR_CUDA;
    cudaDeviceProp prop{};
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return TA_ERR_CUDA;
    if (prop.major != 10) return TA_ERR_UNSUPPORTED;   // sm_100a code only; there is no fallback path
    ta_ctx* c = new (std::nothrow) ta_ctx();
    if (!c) return TA_ERR_NOMEM;
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    if (cudaMalloc(&c->d_status, sizeof(int)) != cudaSuccess || cudaMemset(c->d_status, 0, sizeof(int)) != cudaSuccess) {
        delete c;
        return TA_ERR_CUDA;
    }
    c->ws_owned = true;
    *out = c;
    return TA_OK;
}

int ta_ctx_destroy(ta_ctx* ctx) {
    if (!ctx) return TA_OK;
    cudaSetDevice(ctx->device);
    cudaDeviceSynchronize();
    if (ctx->ws && ctx->ws_owned) cudaFree(ctx->ws);
    if (ctx->d_status) cudaFree(ctx->d_status);
    delete ctx;
    return TA_OK;
}

int ta_ctx_set_workspace(ta_ctx* ctx, void* ws, size_t bytes) {
    if (!ctx) return TA_ERR_INVALID;
    if (ctx->ws && ctx->ws_owned) {
        cudaDeviceSynchronize();
        cudaFree(ctx->ws);
    }
    ctx->ws = ws;
    ctx->ws_bytes = ws ? bytes : 0;
    ctx->ws_owned = (ws == nullptr);
    return TA_OK;
}

const char* ta_last_error(const ta_ctx* ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }

int ta_device_status(ta_ctx* ctx, int* status) {
    if (!ctx || !status) return TA_ERR_INVALID;
    TA_CUDA(ctx, cudaMemcpy(status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (*status != 0) {
        ctx->last_error = *status == 105 ? std::string("a kernel refused its launch shape (status 105)")
                                         : "a bounded device wait ran out (status " + std::to_string(*status) + ")";
        cudaMemset(ctx->d_status, 0, sizeof(int));
        return TA_ERR_DEVICE_TIMEOUT;
    }
    return TA_OK;
}

int ta_ctx_set_gemm_raster(ta_ctx* ctx, int group_m, int group_n) {
    if (!ctx || group_m < 0 || group_n < 0) return TA_ERR_INVALID;
    ctx->gemm_group_m = group_m;
    ctx->gemm_group_n = group_n;
    return TA_OK;
}

long ta_launch_count(const ta_ctx* ctx) { return ctx ? ctx->launches : 0; }

int ta_ctx_set_gemm_tuning(ta_ctx* ctx, int tile_n, int tile_m_halves, int cta_pair) {
    if (!ctx) return TA_ERR_INVALID;
    const bool none = tile_n == 0 && tile_m_halves == 0;
    const bool ok = (tile_m_halves == 1 || tile_m_halves == 2) &&
                    (tile_n == 64 || tile_n == 128 || tile_n == 224 || tile_n == 256) && (tile_m_halves == 1 || tile_n >= 224);
    if (!none && !ok) return ta::fail(ctx, TA_ERR_INVALID, "gemm tuning: tile_n in {64,128,224,256}, halves 1 or 2 (2 needs tile_n >= 224)");
    ctx->gemm_force_bn = tile_n;
    ctx->gemm_force_mh = tile_m_halves;
    if (cta_pair < -1 || cta_pair > 3) return ta::fail(ctx, TA_ERR_INVALID, "gemm tuning: cta_pair in {-1, 0, 1, 2, 3}");
    ctx->gemm_pair = cta_pair;
    return TA_OK;
}

int ta_profile_enable(ta_ctx* ctx, int on) {
    if (!ctx) return TA_ERR_INVALID;
    ctx->profiling = on != 0;
    return TA_OK;
}

int ta_profile_read(ta_ctx* ctx, int n_classes, long* launches, double* work, double* ms) {
    if (!ctx || !launches || !work || !ms || n_classes < ta::PROF_CLASSES) return TA_ERR_INVALID;
    TA_CUDA(ctx, cudaDeviceSynchronize());
    for (int i = 0; i < n_classes; i++) { launches[i] = 0; work[i] = 0; ms[i] = 0; }
    for (auto& r : ctx->prof) {
        float t = 0.f;
        if (cudaEventElapsedTime(&t, r.e0, r.e1) == cudaSuccess) {
            launches[r.cls]++; work[r.cls] += r.work; ms[r.cls] += t;
        }
        cudaEventDestroy(r.e0); cudaEventDestroy(r.e1);
    }
    ctx->prof.clear();
    return TA_OK;
}

}  // extern "C"
