"""HBM-bound kernels through the C ABI vs the NumPy oracle (oracle/ta_oracle.py) on the same seeded
inputs.  Outputs are BF16: the bar is agreement within one BF16 ulp of the oracle value
(|err| <= 2^-7 * |ref| + tiny), because the oracle and the kernel may round a tie differently after
FP32 operations in a different order; exact copies (embedding gather) must be bit-exact."""
import numpy as np
import pytest
import torch

import ta_oracle as o
from tensor_adapt_b200 import ptr, stream_ptr

pytestmark = pytest.mark.gpu


def dev_bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda().to(torch.bfloat16)


def host(t):
    return t.float().cpu().numpy()


def close_bf16(out, ref, ulps=1.0, atol=1e-6):
    tol = ulps * (2.0 ** -7) * np.abs(ref) + atol
    bad = np.abs(out - ref) > tol
    assert not bad.any(), f"{bad.sum()} mismatches, worst {np.abs(out - ref).max()}"


@pytest.mark.parametrize("rows,D", [(37, 896), (64, 3584), (5, 64), (3, 8200 - 8)])
def test_rms_norm_fwd_bwd(ctx, rows, D):
    rng = np.random.default_rng(0)
    x = o.bf16_round(rng.standard_normal((rows, D), dtype=np.float32))
    w = o.bf16_round(1 + 0.1 * rng.standard_normal(D, dtype=np.float32))
    dy = o.bf16_round(rng.standard_normal((rows, D), dtype=np.float32))
    ref_out, ref_rms = o.rms_norm_fwd(x, w, 1e-6)
    xd, wd, dyd = dev_bf16(x), dev_bf16(w), dev_bf16(dy)
    out = torch.empty_like(xd)
    rms = torch.empty(rows, device="cuda", dtype=torch.float32)
    ctx.call("ta_rms_norm_fwd", ptr(xd), ptr(wd), ptr(out), ptr(rms), rows, D, 1e-6, stream_ptr())
    torch.cuda.synchronize()
    np.testing.assert_allclose(rms.cpu().numpy(), ref_rms, rtol=1e-5)
    close_bf16(host(out), ref_out)
    ref_dx = o.rms_norm_bwd(dy, x, w, ref_rms)
    dx = torch.empty_like(xd)
    ctx.call("ta_rms_norm_bwd", ptr(dyd), ptr(xd), ptr(wd), ptr(rms), ptr(dx), None, rows, D, stream_ptr())
    torch.cuda.synchronize()
    close_bf16(host(dx), ref_dx, ulps=1.0, atol=2e-3 * np.abs(ref_dx).max())
    # fused residual-gradient add
    g = o.bf16_round(rng.standard_normal((rows, D), dtype=np.float32))
    gd = dev_bf16(g)
    ctx.call("ta_rms_norm_bwd", ptr(dyd), ptr(xd), ptr(wd), ptr(rms), ptr(gd), ptr(gd), rows, D, stream_ptr())
    torch.cuda.synchronize()
    close_bf16(host(gd), o.add_inplace(g, ref_dx), ulps=1.0, atol=4e-3 * np.abs(ref_dx).max())


@pytest.mark.parametrize("B,T,Hq,Hk,hd", [(2, 33, 14, 2, 64), (1, 130, 4, 2, 128)])
def test_rope_fwd_bwd(ctx, B, T, Hq, Hk, hd):
    rng = np.random.default_rng(1)
    q = o.bf16_round(rng.standard_normal((B * T, Hq * hd), dtype=np.float32))
    k = o.bf16_round(rng.standard_normal((B * T, Hk * hd), dtype=np.float32))
    for inverse in (0, 1):
        qd, kd = dev_bf16(q), dev_bf16(k)
        ctx.call("ta_rope", ptr(qd), Hq, ptr(kd), Hk, B, T, hd, 1e6, inverse, stream_ptr())
        torch.cuda.synchronize()
        close_bf16(host(qd), o.rope(q, B, T, Hq, hd, 1e6, bool(inverse)), atol=1e-4)
        close_bf16(host(kd), o.rope(k, B, T, Hk, hd, 1e6, bool(inverse)), atol=1e-4)


def test_silu_mul(ctx):
    rng = np.random.default_rng(2)
    n = 8 * 4864
    g = o.bf16_round(2 * rng.standard_normal(n, dtype=np.float32))
    u = o.bf16_round(rng.standard_normal(n, dtype=np.float32))
    d = o.bf16_round(rng.standard_normal(n, dtype=np.float32))
    gd, ud, dd = dev_bf16(g), dev_bf16(u), dev_bf16(d)
    out = torch.empty_like(gd)
    ctx.call("ta_silu_mul_fwd", ptr(gd), ptr(ud), ptr(out), n, stream_ptr())
    dg, du = torch.empty_like(gd), torch.empty_like(gd)
    ctx.call("ta_silu_mul_bwd", ptr(dd), ptr(gd), ptr(ud), ptr(dg), ptr(du), n, stream_ptr())
    torch.cuda.synchronize()
    close_bf16(host(out), o.silu_mul_fwd(g, u))
    rg, ru = o.silu_mul_bwd(d, g, u)
    close_bf16(host(dg), rg)
    close_bf16(host(du), ru)


def test_embed_adds_casts(ctx):
    rng = np.random.default_rng(3)
    V, D, BT = 300, 896, 77
    table = o.bf16_round(rng.standard_normal((V, D), dtype=np.float32))
    tok = rng.integers(0, V, BT).astype(np.int32)
    td, tokd = dev_bf16(table), torch.from_numpy(tok).cuda()
    out = torch.empty((BT, D), device="cuda", dtype=torch.bfloat16)
    ctx.call("ta_embed_fwd", ptr(td), ptr(tokd), ptr(out), BT, D, stream_ptr())
    torch.cuda.synchronize()
    assert np.array_equal(host(out), o.embed_fwd(table, tok))          # a copy: bit-exact
    a = o.bf16_round(rng.standard_normal((BT, D), dtype=np.float32))
    b = o.bf16_round(rng.standard_normal((BT, D), dtype=np.float32))
    bias = o.bf16_round(rng.standard_normal(D, dtype=np.float32))
    ad, bd = dev_bf16(a), dev_bf16(b)
    ctx.call("ta_add_inplace", ptr(ad), ptr(bd), BT * D, stream_ptr())
    torch.cuda.synchronize()
    assert np.array_equal(host(ad), o.add_inplace(a, b))               # one FP32 add + RNE: bit-exact
    ad = dev_bf16(a)
    ctx.call("ta_lora_add", ptr(ad), ptr(bd), 2.0, BT * D, stream_ptr())
    torch.cuda.synchronize()
    assert np.array_equal(host(ad), o.lora_add(a, b, 2.0))
    ad, biasd = dev_bf16(a), dev_bf16(bias)
    ctx.call("ta_add_bias", ptr(ad), ptr(biasd), BT, D, stream_ptr())
    torch.cuda.synchronize()
    assert np.array_equal(host(ad), o.add_bias(a, bias))
    f = torch.empty(BT * D + 3, device="cuda", dtype=torch.float32)
    src = dev_bf16(rng.standard_normal(BT * D + 3, dtype=np.float32))
    ctx.call("ta_cast_bf16_to_f32", ptr(src), ptr(f), BT * D + 3, stream_ptr())
    back = torch.empty_like(src)
    ctx.call("ta_cast_f32_to_bf16", ptr(f), ptr(back), BT * D + 3, stream_ptr())
    torch.cuda.synchronize()
    assert torch.equal(f, src.float()) and torch.equal(back, src)


@pytest.mark.parametrize("rows,V", [(19, 151936), (4, 512), (3, 8)])
def test_cross_entropy(ctx, rows, V):
    rng = np.random.default_rng(4)
    logits = o.bf16_round(3 * rng.standard_normal((rows, V), dtype=np.float32))
    tgt = rng.integers(0, V, rows).astype(np.int32)
    tgt[0] = -1                                                         # masked token, reference semantics
    ref_loss, ref_d = o.cross_entropy_fwd(logits, tgt)
    ld, td = dev_bf16(logits), torch.from_numpy(tgt).cuda()
    loss = torch.empty(rows, device="cuda", dtype=torch.float32)
    dl = torch.empty_like(ld)
    ctx.call("ta_cross_entropy_fwd", ptr(ld), ptr(td), ptr(loss), ptr(dl), rows, V, 1.0 / rows, stream_ptr())
    torch.cuda.synchronize()
    np.testing.assert_allclose(loss.cpu().numpy(), ref_loss, rtol=2e-5, atol=2e-5)
    close_bf16(host(dl), ref_d, ulps=1.0, atol=1e-7)
    # in place over the logits, and loss only
    ctx.call("ta_cross_entropy_fwd", ptr(ld), ptr(td), ptr(loss), ptr(ld), rows, V, 1.0 / rows, stream_ptr())
    torch.cuda.synchronize()
    assert torch.equal(ld, dl)


@pytest.mark.parametrize("BT,H,V,chunk", [(200, 128, 1000, 64), (96, 256, 4096, 96), (33, 64, 520, 1000)])
def test_lmhead_ce_fwd_bwd_chunked(ctx, BT, H, V, chunk):
    """lm head + cross-entropy + head backward through a chunk buffer equals the oracle's three
    reference calls on the whole batch (ragged last chunk, chunk larger than the batch)."""
    rng = np.random.default_rng(BT)
    x = o.bf16_round(rng.standard_normal((BT, H), dtype=np.float32))
    W = o.bf16_round(0.05 * rng.standard_normal((V, H), dtype=np.float32))
    tgt = rng.integers(0, V, BT).astype(np.int32)
    tgt[::7] = -1
    logits = o.proj_fwd(W, x)
    ref_loss, ref_d = o.cross_entropy_fwd(logits, tgt)
    inv = 1.0 / 4096                                                     # a global-batch scale, not 1/BT
    ref_dx = o.proj_bwd_x(W, o.bf16_round(ref_d * np.float32(BT * inv)))
    xd, Wd, td = dev_bf16(x), dev_bf16(W), torch.from_numpy(tgt).cuda()
    loss = torch.empty(BT, device="cuda"); dx = torch.empty_like(xd)
    buf = torch.empty(min(chunk, BT) if chunk < BT else chunk, V, device="cuda", dtype=torch.bfloat16)
    ctx.call("ta_lmhead_ce_fwd_bwd", ptr(xd), ptr(Wd), ptr(td), ptr(loss), ptr(dx), BT, H, V, inv, ptr(buf), chunk, stream_ptr())
    torch.cuda.synchronize()
    np.testing.assert_allclose(loss.cpu().numpy(), ref_loss, rtol=3e-5, atol=3e-5)
    assert np.abs(host(dx) - ref_dx).max() <= 2.0 ** -6 * np.abs(ref_dx).max() + 1e-9
