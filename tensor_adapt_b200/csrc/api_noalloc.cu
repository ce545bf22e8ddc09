// Token-contracted LoRA-gradient GEMM for callers that must not allocate.
//
// Who needs this: code that runs where device allocation is forbidden or unsafe - a latency-critical
// loop whose owner has handed out all of device memory to its own pool, or a plugin host that
// pre-sizes memory and treats any cudaMalloc (which also synchronises the whole device) as an error.  The regular entry point ta_gemm_tokens_f32 keeps
// its split-K partials in the context workspace, which is grown with cudaMalloc on demand; this
// variant keeps them in a fixed array that is part of the library image instead.
//
// The price is a hard size limit and a standing cost: every GPU that loads the library holds
// TA_STATIC_SCRATCH_BYTES of device memory until the process exits, whether or not this entry point
// is ever called.
#include "seg_gemm.h"

namespace {

// Split-K partials: [splits][M][N] FP32.  File-scope device storage; its address is only meaningful
// on the device, so host code obtains it with cudaGetSymbolAddress (per device) and never passes the
// symbol itself to a kernel.
static __device__ __align__(256) float g_static_splitk[TA_STATIC_SCRATCH_BYTES / sizeof(float)];

// Written once per device on first use, unsynchronised: contexts are used from one host thread at a time.
constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {};

}  // namespace

extern "C" int ta_gemm_tokens_f32_static(ta_ctx* ctx, int M, int N, int K, float alpha, const void* A, long lda,
                                         const void* B, long ldb, float* C, long ldc, int accumulate, int transpose_out,
                                         void* stream) {
    using namespace ta;
    if (!ctx) return TA_ERR_INVALID;
    if (M <= 0 || N <= 0 || K <= 0) return fail(ctx, TA_ERR_INVALID, "gemm_tokens_f32_static: M, N, K must be > 0");
    int cur = -1;
    TA_CUDA(ctx, cudaGetDevice(&cur));
    if (cur != ctx->device || cur < 0 || cur >= kMaxDevices)
        return fail(ctx, TA_ERR_INVALID, "gemm_tokens_f32_static: the context's device must be the current device");
    if (!g_scratch_ptr[cur]) {
        // one-time set-up for this device (with it current): resolve the device address of the array
        float* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_splitk);
        if (e != cudaSuccess || !p) return check_cuda(ctx, e == cudaSuccess ? cudaErrorUnknown : e, "cudaGetSymbolAddress(static scratch)");
        g_scratch_ptr[cur] = p;
    }
    const int splits = tokens_gemm_splits(ctx, M, N, K);
    const size_t need = size_t(splits) * size_t(M) * size_t(N) * sizeof(float);
    if (need > TA_STATIC_SCRATCH_BYTES)
        return fail(ctx, TA_ERR_NOMEM,
                    "gemm_tokens_f32_static: " + std::to_string(splits) + " splits x " + std::to_string(M) + " x " +
                        std::to_string(N) + " FP32 partials need " + std::to_string(need) + " bytes, the static scratch holds " +
                        std::to_string(size_t(TA_STATIC_SCRATCH_BYTES)) + "; use ta_gemm_tokens_f32 for this size");
    GemmSegment s;
    s.A = static_cast<const __nv_bfloat16*>(A); s.lda = lda; s.a_mn = true;
    s.B = static_cast<const __nv_bfloat16*>(B); s.ldb = ldb; s.b_mn = true;
    s.K = K;
    GemmOut o;
    o.C = C; o.ldc = ldc; o.alpha = alpha; o.f32 = true; o.accumulate = accumulate != 0;
    o.transpose_out = transpose_out != 0;
    o.split_k = splits;
    o.split_ws = g_scratch_ptr[cur];
    o.split_ws_bytes = TA_STATIC_SCRATCH_BYTES;
    o.no_host_state = true;   // tensor maps are encoded on the stack: nothing is inserted into the cache
    // Every partial element [split][m < M][n < N] is written by the GEMM before the reduce reads it, so
    // nothing left over from an earlier call needs clearing.
    return seg_gemm(ctx, static_cast<cudaStream_t>(stream), M, N, &s, 1, o);
}
