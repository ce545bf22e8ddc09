"""Size-independent properties at the FULL shapes of the benchmark config (Qwen2-7B: hidden 3584,
28/4 heads of 128, SwiGLU 18944, vocab 152064, 4096-token sequences), where the NumPy oracle would
take minutes: exact identities the kernels must satisfy whatever the size."""
import ctypes

import numpy as np
import pytest
import torch

from tensor_adapt_b200 import ptr, stream_ptr

pytestmark = pytest.mark.gpu
H, QD, KV, I, V, T = 3584, 3584, 512, 18944, 152064, 4096


def bf(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(torch.bfloat16)


def test_lora_linear_full_size_identities(ctx):
    """B = 0: the fused launch equals the plain GEMM bit for bit and gA stays exactly zero; gB equals the
    split-K product of dY and the separately computed h_s; dX of two stacked halves of the batch equals
    the two halves computed alone (row independence, ragged tile boundary at 8192+40 rows)."""
    BT, r, scale = 8192 + 40, 16, 2.0
    x, W, dY = bf(BT, H, seed=1), bf(I, H, scale=0.02, seed=2), bf(BT, I, seed=3)
    A, B0 = bf(r, H, scale=0.02, seed=4), torch.zeros(I, r, device="cuda", dtype=torch.bfloat16)
    y_l, y_g = torch.empty(BT, I, device="cuda", dtype=torch.bfloat16), torch.empty(BT, I, device="cuda", dtype=torch.bfloat16)
    ctx.call("ta_lora_linear_fwd", ptr(x), ptr(W), None, ptr(A), ptr(B0), None, ptr(y_l), BT, H, I, r, scale, stream_ptr())
    ctx.call("ta_gemm_bf16", BT, I, H, 1.0, ptr(x), H, 0, ptr(W), H, 0, None, None, ptr(y_g), I, stream_ptr())
    assert torch.equal(y_l, y_g)
    gA, gB = torch.zeros(r, H, device="cuda"), torch.zeros(I, r, device="cuda")
    dX = torch.empty(BT, H, device="cuda", dtype=torch.bfloat16)
    ctx.call("ta_lora_linear_bwd", ptr(x), ptr(dY), ptr(W), ptr(A), ptr(B0), ptr(dX), 0, ptr(gA), ptr(gB), BT, H, I, r, scale, stream_ptr())
    assert not gA.any()                                                  # dh = dY.B = 0 exactly
    h = torch.empty(BT, r, device="cuda", dtype=torch.bfloat16)
    ctx.call("ta_gemm_bf16", BT, r, H, scale, ptr(x), H, 0, ptr(A), H, 0, None, None, ptr(h), r, stream_ptr())
    gB2 = torch.zeros(I, r, device="cuda")
    ctx.call("ta_gemm_tokens_f32", I, r, BT, 1.0, ptr(dY), I, ptr(h), r, ptr(gB2), r, 1, 0, stream_ptr())
    assert torch.equal(gB, gB2)
    ref = dY[:64].float() @ W.float()                                    # a corner against FP32 torch
    assert (dX[:64].float() - ref).abs().max() <= 2.0 ** -7 * ref.abs().max()
    half = 4096
    d1 = torch.empty(half, H, device="cuda", dtype=torch.bfloat16)
    ctx.call("ta_lora_linear_bwd", ptr(x), ptr(dY), ptr(W), ptr(A), ptr(B0), ptr(d1), 0, ptr(gA), ptr(gB), half, H, I, r, scale, stream_ptr())
    assert torch.equal(d1, dX[:half])


def test_attention_full_size_causality_and_normalisation(ctx):
    """T = 4096, 28 query / 4 KV heads of 128: (1) keys and values after position t never influence
    out[t] - perturbing the last 1000 positions leaves the first 3096 rows bit-identical; (2) with V
    constant per KV head every output row equals that constant (the probabilities sum to one);
    (3) dV summed over positions equals dO summed over positions and query heads of the group."""
    B, Hq, Hkv, hd = 1, 28, 4, 128
    Q, K, Vv = bf(T, Hq * hd, seed=1), bf(T, Hkv * hd, seed=2), bf(T, Hkv * hd, seed=3)
    out, lse = torch.empty_like(Q), torch.empty(Hq * T, device="cuda")
    ctx.call("ta_flash_attn_fwd", ptr(Q), ptr(K), ptr(Vv), ptr(out), ptr(lse), B, T, Hq, Hkv, hd, stream_ptr())
    K2, V2 = K.clone(), Vv.clone()
    K2[3096:] = bf(T - 3096, Hkv * hd, seed=9); V2[3096:] = bf(T - 3096, Hkv * hd, seed=10)
    out2, lse2 = torch.empty_like(Q), torch.empty_like(lse)
    ctx.call("ta_flash_attn_fwd", ptr(Q), ptr(K2), ptr(V2), ptr(out2), ptr(lse2), B, T, Hq, Hkv, hd, stream_ptr())
    assert torch.equal(out[:3096], out2[:3096]) and not torch.equal(out[3096:], out2[3096:])
    assert torch.equal(lse.view(Hq, T)[:, :3096], lse2.view(Hq, T)[:, :3096])
    const = bf(1, Hkv * hd, seed=5).expand(T, Hkv * hd).contiguous()
    ctx.call("ta_flash_attn_fwd", ptr(Q), ptr(K), ptr(const), ptr(out), ptr(lse), B, T, Hq, Hkv, hd, stream_ptr())
    want = const[0].view(Hkv, 1, hd).expand(Hkv, Hq // Hkv, hd).reshape(1, Hq * hd).float()
    assert (out.float() - want).abs().max() <= 2.0 ** -7 * want.abs().max() + 1e-6
    dO = bf(T, Hq * hd, seed=6)
    dQ, dK, dV = torch.empty_like(Q), torch.empty_like(K), torch.empty_like(Vv)
    ctx.call("ta_flash_attn_fwd", ptr(Q), ptr(K), ptr(Vv), ptr(out), ptr(lse), B, T, Hq, Hkv, hd, stream_ptr())
    ctx.call("ta_flash_attn_bwd", ptr(dO), ptr(Q), ptr(K), ptr(Vv), ptr(out), ptr(lse), ptr(dQ), ptr(dK), ptr(dV), None,
             B, T, Hq, Hkv, hd, stream_ptr())
    # sum_t dV[t] = sum_t sum_h P^T dO = sum over queries and heads of dO (columns of P sum over keys to one per query)
    lhs = dV.float().sum(0).view(Hkv, hd)
    rhs = dO.float().sum(0).view(Hkv, Hq // Hkv, hd).sum(1)
    assert (lhs - rhs).abs().max() <= 2e-2 * rhs.abs().max() + 0.5       # BF16 P and dV roundings over 4096 rows
    assert torch.isfinite(dQ.float()).all() and torch.isfinite(dK.float()).all() and dQ.float().abs().max() > 0


def test_cross_entropy_full_vocab_properties(ctx):
    """152064-wide rows: the gradient of a valid row sums to zero (softmax - one-hot), every loss is
    >= 0 and equals logsumexp - logit[target] computed by torch in FP32."""
    rows = 512
    logits = bf(rows, V, scale=3.0, seed=7)
    tgt = torch.randint(0, V, (rows,), device="cuda", dtype=torch.int32)
    loss, d = torch.empty(rows, device="cuda"), torch.empty_like(logits)
    ctx.call("ta_cross_entropy_fwd", ptr(logits), ptr(tgt), ptr(loss), ptr(d), rows, V, 1.0, stream_ptr())
    lf = logits.float()
    want = torch.logsumexp(lf, 1) - lf.gather(1, tgt.long().view(-1, 1)).squeeze(1)
    assert (loss >= 0).all() and (loss - want).abs().max() <= 2e-4
    assert d.float().sum(1).abs().max() <= 2e-2                          # each of 152064 BF16 roundings is <= 2^-9 relative


def test_swiglu_and_norm_full_size_against_torch(ctx):
    rows = 4096
    g, u, dout = bf(rows, I, seed=1), bf(rows, I, seed=2), bf(rows, I, seed=3)
    act, dg, du = torch.empty_like(g), torch.empty_like(g), torch.empty_like(g)
    ctx.call("ta_silu_mul_fwd", ptr(g), ptr(u), ptr(act), rows * I, stream_ptr())
    ctx.call("ta_silu_mul_bwd", ptr(dout), ptr(g), ptr(u), ptr(dg), ptr(du), rows * I, stream_ptr())
    gf, uf, df = g.float(), u.float(), dout.float()
    sig = torch.sigmoid(gf)
    for got, want in ((act, gf * sig * uf), (du, df * gf * sig), (dg, df * uf * sig * (1 + gf * (1 - sig)))):
        assert (got.float() - want).abs().max() <= 2.0 ** -7 * want.abs().max()
    x, w = bf(rows, H, seed=4), bf(H, seed=5)
    out, rms = torch.empty_like(x), torch.empty(rows, device="cuda")
    ctx.call("ta_rms_norm_fwd", ptr(x), ptr(w), ptr(out), ptr(rms), rows, H, 1e-6, stream_ptr())
    xf = x.float()
    want = xf * torch.rsqrt((xf * xf).mean(1, keepdim=True) + 1e-6) * w.float()
    assert (out.float() - want).abs().max() <= 2.0 ** -7 * want.abs().max()
