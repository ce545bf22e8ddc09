"""Exact-arithmetic arbiter for the LoRA training step.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

The reference (src/base/arch/qwen2.cu:47-308, src/adapter/adapter_model.cu:96-220) and the CUDA library
both compute in BF16 with FP32 accumulation, but round at different points, so comparing one against
the other cannot say which of the two is closer to the mathematical result.  This module evaluates the
same step with torch autograd in FLOAT64 and NO rounding of any intermediate (the inputs - BF16 weights,
BF16 working copies of the LoRA matrices, token ids - are taken as given), which gives the value both
implementations approximate:

    loss, every gA / gB, and the Centroid Accumulator sums  C = sum_t h_t * ||dL/dh_t||

It also carries an EMULATION of the library's rounding points (`Rounding`): BF16 rounding of stored
activations and gradients, of the rank-r activations h / dh, and of the attention probabilities P and
their gradient dS.  Each class can be switched off separately, which attributes the library's distance
from the exact result to its sources (BF16 P / dS inside attention against everything else).

Formulas follow the reference op for op: adjacent-pair RoPE (src/backend/cuda/ops.cu:176-204), LoRA delta
added before RoPE (qwen2.cu:104-111), causal GQA softmax attention with scale 1/sqrt(head_dim)
(ops.cu:578-907), SwiGLU (ops.cu:913-952), cross-entropy with gradient (softmax - onehot) / rows
(ops.cu:958-1020), loss reported as the mean of per-token losses (src/trainer/adapt_trainer.cu:237-246),
centroid accumulation on the input-norm output and its gradient (adapt_trainer.cu:210-232,
src/centroid/centroid_accumulator.cpp:54-69).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch
from torch.utils.checkpoint import checkpoint


@dataclass
class Rounding:
    """Which BF16 roundings of the CUDA library to emulate (all off = exact arithmetic)."""
    acts: bool = False        # stored activations and their gradients (every tensor the library keeps in BF16)
    lora_h: bool = False      # h = bf16(s.x.A^T) and dh = bf16(s.dY.B)
    attn_p: bool = False      # probabilities rounded to BF16 for P.V and P^T.dO
    attn_ds: bool = False     # dS rounded to BF16 for dQ and dK

    @classmethod
    def library(cls):
        return cls(True, True, True, True)

    @classmethod
    def library_fp32_attention(cls):
        return cls(True, True, False, False)


class _RoundFwd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return x.to(torch.bfloat16).to(x.dtype)

    @staticmethod
    def backward(ctx, g):
        return g


class _RoundBwd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return g.to(torch.bfloat16).to(g.dtype)


def _stored(x, on):
    """A tensor the library keeps in BF16: the value is rounded, and so is the gradient that arrives at it."""
    return _RoundBwd.apply(_RoundFwd.apply(x)) if on else x


def _rope(x, B, T, heads, hd, theta):
    xv = x.view(B, T, heads, hd // 2, 2)
    i = torch.arange(hd // 2, device=x.device, dtype=torch.float64)
    ang = torch.arange(T, device=x.device, dtype=torch.float64)[:, None] * torch.pow(torch.tensor(theta, dtype=torch.float64, device=x.device), -2.0 * i / hd)[None, :]
    cs, sn = torch.cos(ang).to(x.dtype)[None, :, None, :], torch.sin(ang).to(x.dtype)[None, :, None, :]
    x0, x1 = xv[..., 0], xv[..., 1]
    return torch.stack([x0 * cs - x1 * sn, x0 * sn + x1 * cs], dim=-1).view(B * T, heads * hd)


def _rms_norm(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * w


def _attention(Q, K, V, B, T, hq, hkv, hd, rnd: Rounding):
    rep = hq // hkv
    q = Q.view(B, T, hq, hd).transpose(1, 2)
    k = K.view(B, T, hkv, hd).transpose(1, 2).repeat_interleave(rep, dim=1)
    v = V.view(B, T, hkv, hd).transpose(1, 2).repeat_interleave(rep, dim=1)
    S = (q @ k.transpose(-1, -2)) * (1.0 / math.sqrt(hd))
    if rnd.attn_ds:
        S = _RoundBwd.apply(S)
    mask = torch.ones(T, T, dtype=torch.bool, device=Q.device).triu(1)
    P = torch.softmax(S.masked_fill(mask, float("-inf")), dim=-1)
    if rnd.attn_p:
        P = _RoundFwd.apply(P)
    return (P @ v).transpose(1, 2).reshape(B * T, hq * hd)


def run_step(cfg, base, adapter, tokens, targets, B, T, scale, rnd: Rounding | None = None, dtype=torch.float64,
             device="cuda", head_chunk=2048):
    """One forward + backward of the LoRA-adapted model.

    cfg / base / adapter are the objects of oracle/ta_oracle.py (BaseConfig, make_base, make_adapter).
    Returns {"loss": mean loss, "grads": {(layer, target): (gA [r,in], gB [out,r])} as float64 NumPy,
    "centroid": {"intended": (acc [H], weight), "asbuilt": (acc [H], weight)}}.
    """
    rnd = rnd or Rounding()
    dev = torch.device(device)
    def t(a):      # NumPy arrays or torch tensors (e.g. BF16 device tensors of a multi-gigabyte base)
        if isinstance(a, torch.Tensor):
            return a.to(device=dev, dtype=dtype)
        return torch.as_tensor(np.ascontiguousarray(a), device=dev).to(dtype)
    H, L = cfg.hidden, cfg.layers
    BT = B * T
    tok = torch.as_tensor(np.asarray(tokens, dtype=np.int64), device=dev)
    tgt = torch.as_tensor(np.asarray(targets, dtype=np.int64), device=dev)
    embed = t(base["embed"])
    lora = {}
    for l in range(L):
        for name, lp in adapter[l].items():
            A = t(lp.A_bf16).requires_grad_(True)
            Bm = t(lp.B_bf16).requires_grad_(True)
            lora[(l, name)] = (A, Bm)

    def proj(l, name, x, W, bias=None):
        y = x @ W.t()
        if bias is not None:
            y = y + bias
        if (l, name) in lora:
            A, Bm = lora[(l, name)]
            h = _stored(scale * (x @ A.t()), rnd.lora_h)
            y = y + h @ Bm.t()
        return y

    r = embed[tok]
    xn_list = []
    for l in range(L):
        w = {k: t(v) for k, v in base["layers"][l].items()}
        r_in = _RoundBwd.apply(r) if rnd.acts else r                # bf16(dx_norm) before it joins the residual gradient
        xn = _stored(_rms_norm(r_in, w["input_norm"], cfg.eps), rnd.acts)
        if xn.requires_grad:
            xn.retain_grad()
        else:                       # layer 0: nothing upstream is trainable, but the centroid needs dL/d(xn)
            xn.requires_grad_(True)
        xn_list.append(xn)
        Q = _stored(proj(l, "q", xn, w["q_w"], w["q_b"]), rnd.acts)
        K = _stored(proj(l, "k", xn, w["k_w"], w["k_b"]), rnd.acts)
        V = _stored(proj(l, "v", xn, w["v_w"], w["v_b"]), rnd.acts)
        Q = _stored(_rope(Q, B, T, cfg.hq, cfg.hd, cfg.theta), rnd.acts)
        K = _stored(_rope(K, B, T, cfg.hkv, cfg.hd, cfg.theta), rnd.acts)
        att = checkpoint(_attention, Q, K, V, B, T, cfg.hq, cfg.hkv, cfg.hd, rnd, use_reentrant=False)
        att = _stored(att, rnd.acts)
        r_mid = _stored(r + proj(l, "o", att, w["o_w"]), rnd.acts)
        rm_in = _RoundBwd.apply(r_mid) if rnd.acts else r_mid
        xn2 = _stored(_rms_norm(rm_in, w["post_norm"], cfg.eps), rnd.acts)
        gate = _stored(proj(l, "gate", xn2, w["gate_w"]), rnd.acts)
        up = _stored(proj(l, "up", xn2, w["up_w"]), rnd.acts)
        act = _stored(torch.nn.functional.silu(gate) * up, rnd.acts)
        r_next = _stored(r_mid + proj(l, "down", act, w["down_w"]), rnd.acts)
        r = r_next
        del w
    rf_in = r
    xf = _stored(_rms_norm(rf_in, t(base["final_norm"]), cfg.eps), rnd.acts)
    lm = embed if cfg.tie else t(base["lm_head"])

    def head(xc, tc):
        logits = _stored(xc @ lm.t(), rnd.acts)
        lse = torch.logsumexp(logits, dim=-1)
        valid = tc >= 0
        tl = torch.where(valid, logits.gather(1, tc.clamp(min=0)[:, None])[:, 0], torch.zeros_like(lse))
        return lse - tl                                                           # per-token loss (ops.cu:997-1001)

    losses = []
    for s in range(0, BT, head_chunk):
        losses.append(checkpoint(head, xf[s:s + head_chunk], tgt[s:s + head_chunk], use_reentrant=False))
    per_token = torch.cat(losses)
    # gradient scale 1 / rows on every token (ops.cu:1005), masked ones included
    (per_token.sum() / BT).backward()
    pos = per_token.detach() > 1e-9
    mean_loss = float(per_token.detach()[pos].sum() / pos.sum()) if bool(pos.any()) else 0.0

    grads = {}
    for (l, name), (A, Bm) in lora.items():
        grads[(l, name)] = (A.grad.double().cpu().numpy(), Bm.grad.double().cpu().numpy())

    acc_i = torch.zeros(H, dtype=torch.float64, device=dev); w_i = torch.zeros((), dtype=torch.float64, device=dev)
    acc_a = torch.zeros(H, dtype=torch.float64, device=dev); w_a = torch.zeros((), dtype=torch.float64, device=dev)
    for xn in xn_list:
        h = xn.detach().double()
        g = xn.grad.double()
        if rnd.acts:
            g = g.to(torch.bfloat16).double()
        gn = g.norm(dim=-1)
        acc_i += (h * gn[:, None]).sum(0); w_i += gn.sum()
        # what the shipped trainer computes (adapt_trainer.cu:215-231 + centroid_accumulator.cpp:45-69): the FP32
        # up-casts re-read as BF16 give rows of D/2 consecutive values of the flat tensor in the odd positions
        h2, g2 = h.reshape(2 * BT, H // 2)[:BT], g.reshape(2 * BT, H // 2)[:BT]
        gn2 = g2.norm(dim=-1)
        acc_a[1::2] += (h2 * gn2[:, None]).sum(0); w_a += gn2.sum()
    return {"loss": mean_loss, "grads": grads,
            "centroid": {"intended": (acc_i.cpu().numpy(), float(w_i)), "asbuilt": (acc_a.cpu().numpy(), float(w_a))}}


def rel_l2(a, b):
    a = np.asarray(a, np.float64).ravel(); b = np.asarray(b, np.float64).ravel()
    return float(np.linalg.norm(a - b) / (np.linalg.norm(b) + 1e-300))


def max_rel(a, b):
    a = np.asarray(a, np.float64); b = np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / (np.abs(b).max() + 1e-300))


def cosine(a, b):
    a = np.asarray(a, np.float64).ravel(); b = np.asarray(b, np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300))
