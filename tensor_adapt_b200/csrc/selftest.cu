// Self-test of the bounded-wait machinery every pipelined kernel of this library relies on: a one-warp kernel
// waits on an mbarrier that nothing will ever arrive at, with a caller-chosen limit of microseconds instead of
// the production 2 s.  No TMA copy, MMA or tensor memory is involved, so giving up leaves nothing in flight: the
// wait must return false, record DS_TIMEOUT_SELFTEST in the context's status word, raise the CTA's abort flag
// (which the other lanes observe) and the kernel must return normally, leaving the CUDA context usable.
#include "ctx.h"
#include "ptx.cuh"

namespace ta {
namespace {

__global__ void bounded_wait_selftest_kernel(int* status, unsigned long long limit_ns, int* observed) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        fence_barrier_init();
    }
    __syncwarp();
    bool ok = true;
    if (threadIdx.x == 0) ok = mbar_wait_limit(&bar, 0, &abort_flag, status, DS_TIMEOUT_SELFTEST, limit_ns);
    __syncwarp();
    // lane 0: 1 if the wait (wrongly) succeeded; lane 1: the abort flag as the rest of the CTA sees it
    if (threadIdx.x == 0) observed[0] = ok ? 1 : 0;
    if (threadIdx.x == 1) observed[1] = *static_cast<volatile int*>(&abort_flag);
}

}  // namespace
}  // namespace ta

extern "C" int ta_selftest_bounded_wait(ta_ctx* ctx, int limit_us, int* wait_returned_true, int* abort_flag_seen, void* stream) {
    if (!ctx || limit_us <= 0 || limit_us > 1000000) return ta::fail(ctx, TA_ERR_INVALID, "selftest: limit_us must be in 1..1000000");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    ta::DeviceBuffer obs;
    TA_CUDA(ctx, obs.alloc(2 * sizeof(int)));
    TA_CUDA(ctx, cudaMemsetAsync(obs.p, 0xFF, 2 * sizeof(int), s));
    ta::bounded_wait_selftest_kernel<<<1, 32, 0, s>>>(ctx->d_status, static_cast<unsigned long long>(limit_us) * 1000ull, obs.as<int>());
    TA_LAUNCH_CHECK(ctx, "bounded_wait_selftest_kernel");
    int h[2] = {-1, -1};
    TA_CUDA(ctx, cudaMemcpyAsync(h, obs.p, sizeof(h), cudaMemcpyDeviceToHost, s));
    TA_CUDA(ctx, cudaStreamSynchronize(s));
    if (wait_returned_true) *wait_returned_true = h[0];
    if (abort_flag_seen) *abort_flag_seen = h[1];
    return TA_OK;
}
