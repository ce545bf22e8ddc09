"""tcgen05 segmented-K GEMM through the C ABI vs a PyTorch FP32 product of the same BF16 operands.

Tolerance: the kernel accumulates in FP32 and rounds once to BF16, so |err| <= 2^-8 * |ref| plus
FP32 summation-order noise; checked as max|err| <= 1e-2 * max|ref| and, for FP32 outputs, 1e-4.
"""
import pytest
import torch

import tensor_adapt_b200 as ta
from tensor_adapt_b200 import ptr, stream_ptr

pytestmark = pytest.mark.gpu


def _mk(shape, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda", dtype=torch.float32) * scale).to(torch.bfloat16)


def _run(ctx, M, N, K, a_mn, b_mn, bias=False, residual=False, alpha=1.0):
    A = _mk((K, M) if a_mn else (M, K), 1)
    B = _mk((K, N) if b_mn else (N, K), 2)
    bias_t = _mk((N,), 3) if bias else None
    res_t = _mk((M, N), 4) if residual else None
    C = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    ctx.call("ta_gemm_bf16", M, N, K, alpha, ptr(A), A.shape[1], int(a_mn), ptr(B), B.shape[1], int(b_mn),
             ptr(bias_t), ptr(res_t), ptr(C), N, stream_ptr())
    torch.cuda.synchronize()
    ctx.check_device()
    Af = A.float().t() if a_mn else A.float()
    Bf = B.float() if b_mn else B.float().t()
    ref = alpha * (Af @ Bf)
    if bias:
        ref = ref + bias_t.float()[None, :]
    if residual:
        ref = ref + res_t.float()
    return C.float(), ref


def _check(out, ref, tol=1e-2):
    assert torch.isfinite(out).all(), "non-finite output (unwritten tile?)"
    err = (out - ref).abs().max().item()
    assert err <= tol * ref.abs().max().item() + 1e-6, f"max err {err} vs ref max {ref.abs().max().item()}"


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 128, 128), (384, 896, 896), (1000, 512, 320)])
def test_gemm_layouts(ctx, M, N, K, a_mn, b_mn):
    out, ref = _run(ctx, M, N, K, a_mn, b_mn)
    _check(out, ref)


@pytest.mark.parametrize("N", [16, 32, 64, 48, 1536])
def test_gemm_narrow_and_ragged_n(ctx, N):
    out, ref = _run(ctx, 520, N, 896, False, False)
    _check(out, ref)
    out, ref = _run(ctx, 520, N, 896, False, True)
    _check(out, ref)


@pytest.mark.parametrize("K", [16, 48, 72, 200])
def test_gemm_ragged_k(ctx, K):
    for a_mn, b_mn in [(False, False), (True, True), (False, True)]:
        out, ref = _run(ctx, 256, 128, K, a_mn, b_mn)
        _check(out, ref)


def test_gemm_epilogue(ctx):
    out, ref = _run(ctx, 4096, 896, 896, False, False, bias=True, residual=True, alpha=0.5)
    _check(out, ref)


def test_gemm_many_tiles_persistent(ctx):
    # more tiles than SMs: exercises the TMEM double buffer and the stage ring across tiles
    out, ref = _run(ctx, 8192, 4864, 896, False, False)
    _check(out, ref)
    out, ref = _run(ctx, 8192, 896, 4864, False, True)
    _check(out, ref)


@pytest.mark.parametrize("M,N,K", [(896, 16, 4096), (4864, 64, 8192), (128, 16, 64), (896, 32, 1000)])
@pytest.mark.parametrize("transpose", [False, True])
def test_gemm_tokens_f32(ctx, M, N, K, transpose):
    A = _mk((K, M), 5)
    B = _mk((K, N), 6)
    shape = (N, M) if transpose else (M, N)
    C0 = torch.randn(shape, device="cuda", dtype=torch.float32)
    C = C0.clone()
    ctx.call("ta_gemm_tokens_f32", M, N, K, 2.0, ptr(A), M, ptr(B), N, ptr(C), shape[1], 1, int(transpose), stream_ptr())
    torch.cuda.synchronize()
    ctx.check_device()
    ref = 2.0 * (A.float().t() @ B.float())
    ref = (ref.t() if transpose else ref) + C0
    err = (C - ref).abs().max().item()
    assert err <= 1e-4 * ref.abs().max().item() + 1e-4, err
    # fixed-order reduction: a second run gives the same bits
    C2 = C0.clone()
    ctx.call("ta_gemm_tokens_f32", M, N, K, 2.0, ptr(A), M, ptr(B), N, ptr(C2), shape[1], 1, int(transpose), stream_ptr())
    torch.cuda.synchronize()
    ctx.call("ta_ctx_set_gemm_tuning", 0, 0, 0)
    assert torch.equal(C, C2)


def test_gemm_rejects_bad_arguments(ctx):
    A = _mk((128, 64), 1)
    with pytest.raises(ta.TAError):
        ctx.call("ta_gemm_bf16", 128, 12, 64, 1.0, ptr(A), 64, 0, ptr(A), 64, 0, None, None, ptr(A), 12, stream_ptr())
    with pytest.raises(ta.TAError):
        ctx.call("ta_gemm_bf16", 128, 64, 64, 1.0, None, 64, 0, ptr(A), 64, 0, None, None, ptr(A), 64, stream_ptr())


@pytest.mark.parametrize("pair_mode", [1, 2, 3])
@pytest.mark.parametrize("M,N,K,b_layout,extras", [(512, 256, 64, 0, False), (1064, 776, 520, 0, False), (1064, 776, 520, 1, False),
                                                     (2048, 1024, 1000, 0, True), (1536, 3584, 1024, 1, True), (300, 264, 4104, 0, True)])
def test_cta_pair_kernel_matches_fp32_reference(ctx, M, N, K, b_layout, extras, pair_mode):
    """The CTA-pair kernels (tcgen05 cta_group::2 over two SMs; mode 1: 512 x 256 pair tiles, mode 2: 256 x 256 pair
    tiles with double-buffered accumulators, mode 3: the same with 128-wide k blocks) against an FP32 torch product: K-major and MN-major B, ragged
    M / N / K, bias and residual."""
    ctx.call("ta_ctx_set_gemm_tuning", 256, 2, pair_mode)
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    A = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    B = (torch.randn((K, N) if b_layout else (N, K), device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    bias = torch.randn(N, device="cuda", generator=g).to(torch.bfloat16) if extras else None
    res = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16) if extras else None
    C = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    ctx.call("ta_gemm_bf16", M, N, K, 1.0, ptr(A), K, 0, ptr(B), B.shape[1], b_layout, ptr(bias) if extras else None,
             ptr(res) if extras else None, ptr(C), N, stream_ptr())
    torch.cuda.synchronize()
    ctx.check_device()
    ref = A.float() @ (B.float() if b_layout else B.float().t())
    if extras:
        ref = ref + bias.float() + res.float()
    assert (C.float() - ref).abs().max() <= 2.0 ** -7 * ref.abs().max() + 1e-3
    # and it is the same result as the single-CTA kernel, bit for bit (same accumulation order per output element)
    ctx.call("ta_ctx_set_gemm_tuning", 256, 2, -1)
    C2 = torch.zeros_like(C)
    ctx.call("ta_gemm_bf16", M, N, K, 1.0, ptr(A), K, 0, ptr(B), B.shape[1], b_layout, ptr(bias) if extras else None,
             ptr(res) if extras else None, ptr(C2), N, stream_ptr())
    torch.cuda.synchronize()
    ctx.call("ta_ctx_set_gemm_tuning", 0, 0, 0)
    assert torch.equal(C, C2)
