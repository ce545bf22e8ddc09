"""SwiGLU folded into the GEMM epilogues: gate/up projection (+ adapters) + silu_mul_fwd as one launch, and the down
projection's dX + silu_mul_bwd as one launch, each against an FP32 torch evaluation of the reference's op sequence
(src/base/arch/qwen2.cu:137-147,221-230; src/backend/cuda/ops.cu:913-941), on both 256-row kernels (single CTA and
CTA pair), with ragged sizes; and the whole training step with the fusion on must agree with the step with it off
(separate kernels, the already-pinned path) to BF16 rounding."""
import numpy as np
import pytest
import torch

import refcase as rc
import tensor_adapt_b200 as ta
from tensor_adapt_b200 import ptr, stream_ptr

pytestmark = pytest.mark.gpu


def _r(shape, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, device="cuda", generator=g) * scale).to(torch.bfloat16)


def _bf(x):
    return x.to(torch.bfloat16).float()


@pytest.mark.parametrize("pair", [-1, 0, 2, 3])
@pytest.mark.parametrize("BT,H,I,rank", [(512, 256, 384, 16), (1064, 520, 1000, 16), (768, 896, 4864, 64), (300, 128, 136, 32),
                                          (640, 256, 512, 0), (2048, 1536, 2048, 48)])
def test_fused_gate_up_swiglu_forward(ctx, BT, H, I, rank, pair):
    x = _r((BT, H), 1)
    Wg, Wu = _r((I, H), 2, 0.05), _r((I, H), 3, 0.05)
    scale = 2.0
    A = _r((2 * rank, H), 4, 0.05) if rank else None
    Bg, Bu = (_r((I, rank), 5, 0.1), _r((I, rank), 6, 0.1)) if rank else (None, None)
    gate, up, act = (torch.zeros(BT, I, device="cuda", dtype=torch.bfloat16) for _ in range(3))
    ctx.call("ta_ctx_set_gemm_tuning", 0, 0, pair)
    ctx.call("ta_swiglu_proj_fwd", ptr(x), ptr(Wg), ptr(Wu), ptr(A) if rank else None, ptr(Bg) if rank else None,
             ptr(Bu) if rank else None, ptr(gate), ptr(up), ptr(act), BT, H, I, rank, scale, stream_ptr())
    torch.cuda.synchronize()
    ctx.call("ta_ctx_set_gemm_tuning", 0, 0, 0)
    ctx.check_device()
    xf = x.float()
    g_ref, u_ref = xf @ Wg.float().t(), xf @ Wu.float().t()
    if rank:
        h = _bf(scale * (xf @ A.float().t()))                       # [BT, 2r], rounded like the library's h_s
        g_ref = g_ref + h[:, :rank] @ Bg.float().t()
        u_ref = u_ref + h[:, rank:] @ Bu.float().t()
    tol = lambda ref: 2.0 ** -7 * ref.abs().max() + 1e-3
    assert (gate.float() - g_ref).abs().max() <= tol(g_ref)
    assert (up.float() - u_ref).abs().max() <= tol(u_ref)
    # act is formed from the ROUNDED gate / up, exactly as the separate kernel reads them
    a_ref = torch.nn.functional.silu(gate.float()) * up.float()
    assert (act.float() - a_ref).abs().max() <= 2.0 ** -8 * a_ref.abs().max() + 1e-6


@pytest.mark.parametrize("pair", [-1, 0, 2, 3])
@pytest.mark.parametrize("BT,H,I,rank", [(512, 256, 384, 16), (1064, 520, 1000, 16), (768, 896, 4864, 0), (300, 128, 136, 32),
                                          (100, 64, 72, 16)])
def test_fused_down_backward_swiglu(ctx, BT, H, I, rank, pair):
    dY, Wd = _r((BT, H), 1), _r((H, I), 2, 0.05)
    gate, up = _r((BT, I), 3), _r((BT, I), 4)
    dh = _r((BT, rank), 5, 0.1) if rank else None
    Ad = _r((rank, I), 6, 0.1) if rank else None
    d_gate, d_up = (torch.zeros(BT, I, device="cuda", dtype=torch.bfloat16) for _ in range(2))
    ctx.call("ta_ctx_set_gemm_tuning", 0, 0, pair)
    ctx.call("ta_swiglu_down_bwd", ptr(dY), ptr(Wd), ptr(dh) if rank else None, ptr(Ad) if rank else None, ptr(gate), ptr(up),
             ptr(d_gate), ptr(d_up), BT, H, I, rank, stream_ptr())
    torch.cuda.synchronize()
    ctx.call("ta_ctx_set_gemm_tuning", 0, 0, 0)
    ctx.check_device()
    d_act = dY.float() @ Wd.float()
    if rank:
        d_act = d_act + dh.float() @ Ad.float()
    g, u = gate.float(), up.float()
    sig = torch.sigmoid(g)
    dg_ref, du_ref = d_act * u * (sig * (1 + g * (1 - sig))), d_act * (g * sig)
    assert (d_gate.float() - dg_ref).abs().max() <= 2.0 ** -7 * dg_ref.abs().max() + 1e-3
    assert (d_up.float() - du_ref).abs().max() <= 2.0 ** -7 * du_ref.abs().max() + 1e-3


def test_fused_forward_rejects_bad_arguments(ctx):
    x, W = _r((128, 64), 1), _r((64, 64), 2)
    out = torch.zeros(128, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ta.TAError):          # fewer than 256 rows: the 256-row tile kernels do not apply
        ctx.call("ta_swiglu_proj_fwd", ptr(x), ptr(W), ptr(W), None, None, None, ptr(out), ptr(out), ptr(out), 128, 64, 64, 0, 1.0,
                 stream_ptr())
    x = _r((256, 64), 1)
    out = torch.zeros(256, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ta.TAError):          # rank must be a multiple of 16
        ctx.call("ta_swiglu_proj_fwd", ptr(x), ptr(W), ptr(W), ptr(W), ptr(W), ptr(W), ptr(out), ptr(out), ptr(out), 256, 64, 64, 8, 1.0,
                 stream_ptr())


@pytest.mark.parametrize("targets", [127, 15, 16 | 64])
def test_training_step_with_fused_swiglu_equals_unfused(ctx, targets):
    """Same step, SwiGLU fused into the GEMM epilogues or run as separate kernels: the forward is bit-identical
    (act is formed from the rounded gate / up either way), gradients differ only by the BF16 rounding of d_act that
    the fused backward skips."""
    from tensor_adapt_b200.trainer import AdaptTrainer, AdapterConfig
    cfg = rc.tiny_cfg(hidden=256, hq=4, hkv=2, hd=64, inter=640, layers=2)
    B, T, rank = 2, 256, 16
    names = [n for b, n in enumerate(("q", "k", "v", "o", "gate", "up", "down")) if targets & (1 << b)]
    base, adapter, toks, tgts = rc.make_case(cfg, B, T, rank, targets=names, seed=31, std=0.02, b_std=0.02)
    res = []
    for fused in (1, 0):
        ac = AdapterConfig.defaults(rank=rank, alpha=32.0, targets=targets, lr=2e-4, centroid_modes=1)
        tr = AdaptTrainer(ctx, rc.model_config(cfg), ac, B, T)
        rc.load_into_trainer(tr, cfg, base, adapter)
        tr._call("ta_trainer_set_option", b"fuse_swiglu", fused)
        tr.zero_grad(); tr.forward_backward(toks[0], tgts[0], B)
        m = tr.optimizer_step(2e-4)
        res.append((m.loss, tr.download("lora.grad"), tr.download("centroid.acc"), ctx.launches))
        ctx.check_device(); tr.close()
    (lf, gf, cf, nf), (lu, gu, cu, nu) = res
    assert lf == lu                                             # forward bit-identical
    assert rc.cosine(gf, gu) >= 0.99999 and np.abs(gf - gu).max() <= 2e-2 * np.abs(gu).max()
    assert np.linalg.norm(cf - cu) <= 1e-3 * np.linalg.norm(cu)
