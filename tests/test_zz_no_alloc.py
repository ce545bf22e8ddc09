"""The allocation-free variant of the token-contracted gradient GEMM (ta_gemm_tokens_f32_static).

Some users of this library run where device allocation is off limits: inside a serving or training
process that has already handed every byte of device memory to its own pool, or behind a plugin
interface that treats cudaMalloc (and the device-wide stall it causes) as a fault.  For them the split-K partials live in a fixed array compiled into the library.  This file
checks, through the C ABI, that the variant returns what the regular entry point returns - twice in a
row, because the array keeps the previous call's contents - that both agree with a plain FP32 product,
and that oversized requests are refused
with a readable message instead of overrunning the array.  It is collected last on purpose."""
import numpy as np
import pytest
import torch

import tensor_adapt_b200 as ta
from tensor_adapt_b200 import ptr, stream_ptr

pytestmark = pytest.mark.gpu


def _mk(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(shape, generator=g, device="cuda").to(torch.bfloat16)


def test_static_scratch_variant_matches_regular_entry_point(ctx):
    # (out features, rank, tokens): the LoRA gradient shapes of the 0.5B config, a ragged one, and a
    # second, smaller problem afterwards so that stale partials of the first would show
    for (M, N, K, transpose) in [(896, 16, 8192, False), (896, 16, 8192, True), (1000, 32, 3000, False), (128, 16, 64, True)]:
        A, B = _mk((K, M), 11), _mk((K, N), 12)
        shape = (N, M) if transpose else (M, N)
        C0 = torch.randn(shape, device="cuda")
        ref = C0.clone()
        ctx.call("ta_gemm_tokens_f32", M, N, K, 2.0, ptr(A), M, ptr(B), N, ptr(ref), shape[1], 1, int(transpose), stream_ptr())
        prod = 2.0 * (A.float().t() @ B.float())                     # [M, N] in plain FP32 arithmetic
        exact = C0 + (prod.t() if transpose else prod)
        for attempt in range(2):
            out = C0.clone()
            ctx.call("ta_gemm_tokens_f32_static", M, N, K, 2.0, ptr(A), M, ptr(B), N, ptr(out), shape[1], 1, int(transpose),
                     stream_ptr())
            torch.cuda.synchronize()
            # same kernels, same split count, same reduction order; the tolerance is the one the
            # regular entry point is tested with
            err = (out - ref).abs().max().item()
            assert err <= 1e-4 * ref.abs().max().item() + 1e-4, (M, N, K, transpose, attempt, err)
            # and on its own feet: against the FP32 product (only the summation order differs)
            assert (out - exact).abs().max().item() <= 1e-3 * exact.abs().max().item(), (M, N, K, transpose, attempt)
    ctx.check_device()


def test_static_scratch_variant_allocates_nothing(ctx):
    M, N, K = 896, 16, 4096
    A, B = _mk((K, M), 1), _mk((K, N), 2)
    C = torch.zeros((M, N), device="cuda")
    ctx.call("ta_gemm_tokens_f32_static", M, N, K, 1.0, ptr(A), M, ptr(B), N, ptr(C), N, 0, 0, stream_ptr())   # set-up call
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        ctx.call("ta_gemm_tokens_f32_static", M, N, K, 1.0, ptr(A), M, ptr(B), N, ptr(C), N, 0, 0, stream_ptr())
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0


def test_static_scratch_variant_rejects_oversized_requests(ctx):
    M, N, K = 18944, 64, 16384          # 7B down-projection gradient at rank 64: partials exceed 8 MiB
    A, B = _mk((K, M), 3), _mk((K, N), 4)
    C = torch.zeros((M, N), device="cuda")
    with pytest.raises(ta.TAError) as e:
        ctx.call("ta_gemm_tokens_f32_static", M, N, K, 1.0, ptr(A), M, ptr(B), N, ptr(C), N, 0, 0, stream_ptr())
    assert "static scratch holds" in str(e.value) and "ta_gemm_tokens_f32" in str(e.value)
    torch.cuda.synchronize()
    assert float(C.abs().max()) == 0.0   # nothing was launched
