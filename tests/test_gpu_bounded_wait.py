"""The give-up path of the bounded device waits, exercised safely: a one-warp kernel (no TMA copy, no MMA, no
tensor memory) waits 2 ms on a barrier that nothing arrives at.  The wait must run out, the kernel must return,
ta_device_status must report TA_ERR_DEVICE_TIMEOUT with the self-test's code - and the CUDA context must be as
usable afterwards as before (a real GEMM still gives the right answer and the status word is clean again)."""
import ctypes
import time

import pytest
import torch

import tensor_adapt_b200 as ta
from tensor_adapt_b200 import ptr, stream_ptr

pytestmark = pytest.mark.gpu


def test_wait_runs_out_is_reported_and_the_context_survives(ctx):
    ctx.check_device()                                           # clean before
    ok, flag = ctypes.c_int(-1), ctypes.c_int(-1)
    t0 = time.perf_counter()
    ctx.call("ta_selftest_bounded_wait", 2000, ctypes.byref(ok), ctypes.byref(flag), stream_ptr())
    dt = time.perf_counter() - t0
    assert ok.value == 0, "the wait on a barrier nobody arrives at must give up"
    assert flag.value == 1, "the CTA-wide abort flag must be visible to the other lanes"
    assert 0.0015 <= dt < 1.0, dt                                 # it waited its limit, not the production 2 s
    st = ctypes.c_int(0)
    rc = ta.lib.ta_device_status(ctx.h, ctypes.byref(st))
    assert rc == -4 and st.value == 106                           # TA_ERR_DEVICE_TIMEOUT, DS_TIMEOUT_SELFTEST
    with_msg = ta.lib.ta_last_error(ctx.h).decode()
    assert "106" in with_msg
    ctx.check_device()                                           # reading the status clears it
    # the context still computes
    g = torch.Generator(device="cuda").manual_seed(1)
    A = torch.randn(256, 128, device="cuda", generator=g).to(torch.bfloat16)
    B = torch.randn(256, 128, device="cuda", generator=g).to(torch.bfloat16)
    C = torch.zeros(256, 256, device="cuda", dtype=torch.bfloat16)
    ctx.call("ta_gemm_bf16", 256, 256, 128, 1.0, ptr(A), 128, 0, ptr(B), 128, 0, None, None, ptr(C), 256, stream_ptr())
    torch.cuda.synchronize()
    ref = A.float() @ B.float().t()
    assert (C.float() - ref).abs().max() <= 2.0 ** -7 * ref.abs().max()
    ctx.check_device()


def test_selftest_rejects_silly_limits(ctx):
    with pytest.raises(ta.TAError):
        ctx.call("ta_selftest_bounded_wait", 0, None, None, stream_ptr())
    with pytest.raises(ta.TAError):
        ctx.call("ta_selftest_bounded_wait", 5_000_000, None, None, stream_ptr())
