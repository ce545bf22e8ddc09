"""CPU restatement of the reference's LoRA training step.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference arm may import this
module; the product path (the CUDA library) never does and has no CPU fallback.

Every function restates one piece of carbon-os/tensor-adapt and cites the file:line it follows
(paths are relative to the reference tree).  Arithmetic follows the reference's rounding points:
tensors that the reference holds in BF16 are FP32 arrays whose values are BF16-representable
(`bf16_round`), reductions are FP32.  cuBLAS calls (`cublasGemmEx` BF16 in/out with FP32
accumulation, `cublasSgemm`, `cublasGemmStridedBatchedEx` FP32) are a closed NVIDIA library,
CUDA 12.9 on this image, not pinned by the reference (BUILD.md says >= 11.8); their contract is an
FP32-accumulated matrix product, restated as a NumPy FP32 matmul (summation order differs, so
GEMM-derived results are compared with tolerances, never bit-for-bit).

Parity pins:
  * k-means merge and both centroid loops: byte-identical to the unmodified reference binary
    oracle/_ref/centroid-merge on the same snapshot files (tests/test_oracle_golden.py), and
    tests/golden/kmeans_cfg1.npz holds the reference binary's output for the 2048 x 512, k = 8 merge case.
  * forward / cross-entropy / backward / AdamW / centroid / checkpoint files: against dumps of the
    unmodified reference objects run by oracle/ref_harness.cu on a B200, committed as
    tests/golden/ref_*.npz together with tests/golden/make_golden.py which made them.
  * LoRA on gate/up/down and seeded k-means++ / mass ranking have no reference implementation:
    "extension, parity unpinned by the reference" - they reuse the formulas pinned above.
"""
from __future__ import annotations

import ctypes
import json
import math
import os
import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
F32 = np.float32


# ───────────────────────────── BF16 helpers ─────────────────────────────

def bf16_bits(x: np.ndarray) -> np.ndarray:
    """FP32 -> BF16 bit pattern (uint16), round-to-nearest-even: what `__float2bfloat16` does
    (src/backend/cuda/ops.cu:1123-1126, src/checkpoint/adapter_writer.cpp:44-47)."""
    u = np.ascontiguousarray(x, dtype=F32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = (u + (((u >> 16) & 1) + np.uint32(0x7FFF))) >> 16
    r = np.where(nan, np.uint32(0x7FFF), r)
    return r.astype(np.uint16)


def bf16_from_bits(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(F32)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """FP32 array -> FP32 array holding the nearest BF16 values."""
    return bf16_from_bits(bf16_bits(x)).reshape(np.shape(x))


# ───────────────────────────── GEMM contracts ─────────────────────────────

def gemm_bf16(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """`gemm_bf16` (src/backend/cuda/tensor.cu:144-166): BF16 operands, FP32 accumulate, BF16 out."""
    return bf16_round(a.astype(F32) @ b.astype(F32))


def proj_fwd(W: np.ndarray, x: np.ndarray) -> np.ndarray:
    """y = x.W^T (src/base/arch/qwen2.cu:21-30). W [out,in], x [BT,in] -> [BT,out] BF16."""
    return gemm_bf16(x, W.T)


def proj_bwd_x(W: np.ndarray, dy: np.ndarray, dx: Optional[np.ndarray] = None) -> np.ndarray:
    """dx = beta.dx + dy.W with a BF16 re-round per call (src/base/arch/qwen2.cu:32-41)."""
    acc = dy.astype(F32) @ W.astype(F32)
    if dx is not None:
        acc = acc + dx
    return bf16_round(acc)


# ───────────────────────────── element-wise / row ops ─────────────────────────────

def rms_norm_fwd(x: np.ndarray, w: np.ndarray, eps: float) -> Tuple[np.ndarray, np.ndarray]:
    """src/backend/cuda/ops.cu:59-107: rms = rsqrt(mean(x^2)+eps); out = bf16(x*rms*w)."""
    x = x.astype(F32)
    ss = np.sum(x * x, axis=-1, dtype=F32)
    rms = (F32(1.0) / np.sqrt(ss / F32(x.shape[-1]) + F32(eps))).astype(F32)
    return bf16_round(x * rms[:, None] * w.astype(F32)[None, :]), rms


def rms_norm_bwd(dy: np.ndarray, x: np.ndarray, w: np.ndarray, rms: np.ndarray) -> np.ndarray:
    """src/backend/cuda/ops.cu:113-170: dx = rms*(w*dy - x_hat*mean(dy*w*x_hat)). The dw atomics
    (:156) are discarded by every caller (src/base/arch/qwen2.cu:207,240,298) and not restated."""
    dy = dy.astype(F32); x = x.astype(F32); w = w.astype(F32)[None, :]
    xh = x * rms[:, None]
    corr = np.sum(dy * w * xh, axis=-1, dtype=F32) / F32(x.shape[-1])
    return bf16_round(rms[:, None] * (w * dy - xh * corr[:, None]))


def rope(x: np.ndarray, B: int, T: int, H: int, hd: int, theta: float, inverse: bool = False) -> np.ndarray:
    """src/backend/cuda/ops.cu:176-204: rotation of ADJACENT pairs (2i, 2i+1), freq = theta^(-2i/hd),
    angle = t*freq (negated for the backward), applied in place on BF16 [BT, H*hd]."""
    xv = x.astype(F32).reshape(B, T, H, hd // 2, 2)
    i = np.arange(hd // 2, dtype=F32)
    freq = np.power(F32(theta), -2.0 * i / F32(hd)).astype(F32)
    ang = (np.arange(T, dtype=F32)[:, None] * freq[None, :]).astype(F32)
    if inverse:
        ang = -ang
    cs = np.cos(ang.astype(np.float64)).astype(F32)[None, :, None, :]
    sn = np.sin(ang.astype(np.float64)).astype(F32)[None, :, None, :]
    x0, x1 = xv[..., 0], xv[..., 1]
    out = np.stack([x0 * cs - x1 * sn, x0 * sn + x1 * cs], axis=-1)
    return bf16_round(out.reshape(B * T, H * hd))


def add_bias(out: np.ndarray, bias: np.ndarray) -> np.ndarray:
    """src/backend/cuda/ops.cu:1062-1081."""
    return bf16_round(out.astype(F32) + bias.astype(F32)[None, :])


def add_inplace(out: np.ndarray, delta: np.ndarray) -> np.ndarray:
    """src/backend/cuda/ops.cu:1087-1099."""
    return bf16_round(out.astype(F32) + delta.astype(F32))


def lora_add(out: np.ndarray, delta: np.ndarray, scale: float) -> np.ndarray:
    """src/backend/cuda/ops.cu:1101-1113."""
    return bf16_round(out.astype(F32) + F32(scale) * delta.astype(F32))


def silu_mul_fwd(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """src/backend/cuda/ops.cu:913-923."""
    g = gate.astype(F32); u = up.astype(F32)
    return bf16_round(g / (F32(1) + np.exp(-g)) * u)


def silu_mul_bwd(dout: np.ndarray, gate: np.ndarray, up: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """src/backend/cuda/ops.cu:925-941."""
    g = gate.astype(F32); u = up.astype(F32); do = dout.astype(F32)
    sig = F32(1) / (F32(1) + np.exp(-g))
    s = g * sig
    ds = sig * (F32(1) + g * (F32(1) - sig))
    return bf16_round(do * u * ds), bf16_round(do * s)


def embed_fwd(table: np.ndarray, tokens: np.ndarray) -> np.ndarray:
    """src/backend/cuda/ops.cu:1026-1036."""
    return table[tokens].astype(F32)


def cross_entropy_fwd(logits: np.ndarray, targets: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """src/backend/cuda/ops.cu:958-1020.  loss = logsumexp - logit[tgt]; for tgt < 0 the target
    logit is taken as 0 so loss = logsumexp (:997-998) and the gradient is still softmax/N
    (:1008-1010): masked tokens are NOT excluded.  N = number of rows (gridDim.x)."""
    L = logits.astype(F32)
    N, V = L.shape
    mx = L.max(axis=-1)
    s = np.sum(np.exp(L - mx[:, None]), axis=-1, dtype=F32)
    lse = (np.log(s) + mx).astype(F32)
    valid = targets >= 0
    tl = np.where(valid, L[np.arange(N), np.where(valid, targets, 0)], F32(0)).astype(F32)
    loss = (-(tl - lse)).astype(F32)
    p = np.exp(L - lse[:, None])
    p[np.arange(N)[valid], targets[valid]] -= F32(1)
    return loss, bf16_round(p * F32(1.0 / N))


# ───────────────────────────── attention ─────────────────────────────

def sdpa_fwd(Q, K, V, B, T, Hq, Hkv, hd):
    """Batched path of ops::sdpa_fwd (src/backend/cuda/ops.cu:578-681): everything in FP32 -
    S = scale.Q.K^T, causal softmax (:352-396), O = P.V, O rounded to BF16 on unpack.
    Returns (out [BT,Hq*hd] BF16, P [B,Hq,T,T] FP32)."""
    q = Q.astype(F32).reshape(B, T, Hq, hd).transpose(0, 2, 1, 3)
    k = K.astype(F32).reshape(B, T, Hkv, hd).transpose(0, 2, 1, 3)
    v = V.astype(F32).reshape(B, T, Hkv, hd).transpose(0, 2, 1, 3)
    rep = Hq // Hkv
    k = np.repeat(k, rep, axis=1); v = np.repeat(v, rep, axis=1)    # k_expand_kv_pack :518-536
    S = (F32(1.0 / math.sqrt(hd)) * (q @ k.transpose(0, 1, 3, 2))).astype(F32)
    mask = np.triu(np.ones((T, T), dtype=bool), 1)
    S = np.where(mask, -np.inf, S)
    S = S - S.max(axis=-1, keepdims=True)
    P = np.exp(S).astype(F32)
    P = (P / P.sum(axis=-1, keepdims=True, dtype=F32)).astype(F32)
    O = (P @ v).astype(F32)
    return bf16_round(O.transpose(0, 2, 1, 3).reshape(B * T, Hq * hd)), P


def sdpa_bwd(dout, Q, K, V, P, B, T, Hq, Hkv, hd):
    """ops::sdpa_bwd batched path (src/backend/cuda/ops.cu:707-870): dV = P^T.dO, dP = dO.V^T,
    dS = P*(dP - sum(P*dP)) (:405-435), dQ = scale.dS.K, dK = scale.dS^T.Q, GQA heads summed in
    FP32 (:539-555) before the BF16 cast."""
    rep = Hq // Hkv
    do = dout.astype(F32).reshape(B, T, Hq, hd).transpose(0, 2, 1, 3)
    q = Q.astype(F32).reshape(B, T, Hq, hd).transpose(0, 2, 1, 3)
    k = np.repeat(K.astype(F32).reshape(B, T, Hkv, hd).transpose(0, 2, 1, 3), rep, axis=1)
    v = np.repeat(V.astype(F32).reshape(B, T, Hkv, hd).transpose(0, 2, 1, 3), rep, axis=1)
    sc = F32(1.0 / math.sqrt(hd))
    dVx = (P.transpose(0, 1, 3, 2) @ do).astype(F32)
    dP = (do @ v.transpose(0, 1, 3, 2)).astype(F32)
    dot = np.sum(P * dP, axis=-1, keepdims=True, dtype=F32)
    dS = (P * (dP - dot)).astype(F32)
    dQ = (sc * (dS @ k)).astype(F32)
    dKx = (sc * (dS.transpose(0, 1, 3, 2) @ q)).astype(F32)
    dK = dKx.reshape(B, Hkv, rep, T, hd).sum(axis=2, dtype=F32)
    dV = dVx.reshape(B, Hkv, rep, T, hd).sum(axis=2, dtype=F32)
    back = lambda a, H: bf16_round(a.transpose(0, 2, 1, 3).reshape(B * T, H * hd))
    return back(dQ, Hq), back(dK, Hkv), back(dV, Hkv)


# ───────────────────────────── LoRA ─────────────────────────────

@dataclass
class LoraPair:
    """src/include: include/tensor/adapter/adapter_model.hpp:26-36.  A [r,in], B [out,r]; F32 masters,
    BF16 working copies derived from them, F32 moments and gradients."""
    A_f32: np.ndarray
    B_f32: np.ndarray
    mA: np.ndarray = None
    vA: np.ndarray = None
    mB: np.ndarray = None
    vB: np.ndarray = None
    gA: np.ndarray = None
    gB: np.ndarray = None

    def __post_init__(self):
        self.A_f32 = np.ascontiguousarray(self.A_f32, dtype=F32)
        self.B_f32 = np.ascontiguousarray(self.B_f32, dtype=F32)
        z = lambda a: np.zeros_like(a, dtype=F32)
        self.mA = z(self.A_f32) if self.mA is None else self.mA
        self.vA = z(self.A_f32) if self.vA is None else self.vA
        self.mB = z(self.B_f32) if self.mB is None else self.mB
        self.vB = z(self.B_f32) if self.vB is None else self.vB
        self.gA = z(self.A_f32) if self.gA is None else self.gA
        self.gB = z(self.B_f32) if self.gB is None else self.gB
        self.A_bf16 = bf16_round(self.A_f32)
        self.B_bf16 = bf16_round(self.B_f32)

    def zero_grad(self):
        self.gA[...] = 0; self.gB[...] = 0


def kaiming_init(in_dim: int, rank: int, seed: int = 0x1234) -> np.ndarray:
    """k_kaiming_init_f32 (src/adapter/adapter_model.cu:28-39): integer-hash uniform in [-1,1] times
    sqrt(1/in_dim); the same seed 0x1234 for every pair (:53-54)."""
    i = np.arange(in_dim * rank, dtype=np.uint64)
    r = (np.uint64(seed) ^ ((i * np.uint64(2654435761)) & np.uint64(0xFFFFFFFF))) & np.uint64(0xFFFFFFFF)
    r = r ^ (r >> np.uint64(16))
    r = (r * np.uint64(0x45d9f3b)) & np.uint64(0xFFFFFFFF)
    r = r ^ (r >> np.uint64(16))
    u = ((r & np.uint64(0xFFFFFF)).astype(F32) / F32(0xFFFFFF) * F32(2) - F32(1)).astype(F32)
    bound = F32(math.sqrt(1.0 / in_dim))
    return (u * bound).astype(F32).reshape(rank, in_dim)


def apply_lora_fwd(lp: LoraPair, x: np.ndarray, out: np.ndarray, scale: float) -> np.ndarray:
    """src/adapter/adapter_model.cu:96-129: h = bf16(x.A^T); delta = bf16(h.B^T); out = bf16(out + s*delta)."""
    h = gemm_bf16(x, lp.A_bf16.T)
    delta = gemm_bf16(h, lp.B_bf16.T)
    return lora_add(out, delta, scale)


def apply_lora_bwd(lp: LoraPair, x: np.ndarray, dY: np.ndarray, dX: np.ndarray, scale: float) -> np.ndarray:
    """src/adapter/adapter_model.cu:131-220: h recomputed and rounded to BF16; gB += s.dY^T.h and
    gA += s.dh^T.x as FP32 GEMMs on up-cast copies; dh = bf16(dY.B); dX = bf16(dX + s.dh.A)."""
    h = gemm_bf16(x, lp.A_bf16.T)
    lp.gB += F32(scale) * (dY.astype(F32).T @ h)
    dh = gemm_bf16(dY, lp.B_bf16)
    lp.gA += F32(scale) * (dh.T @ x.astype(F32))
    return bf16_round(dX.astype(F32) + F32(scale) * (dh @ lp.A_bf16))


# ───────────────────────────── model ─────────────────────────────

@dataclass
class BaseConfig:
    """include/tensor/base/frozen_base.hpp:15-29."""
    vocab: int
    hidden: int
    layers: int
    hq: int
    hkv: int
    hd: int
    inter: int
    eps: float = 1e-6
    theta: float = 1e6
    tie: bool = True


#: projections that can carry a LoRA pair. The reference wires only the first four
#: (src/adapter/adapter_model.cu:82-87); gate/up/down are an extension (the 1.5B and 7B benchmark configurations adapt all seven).
ALL_TARGETS = ("q", "k", "v", "o", "gate", "up", "down")


def make_base(cfg: BaseConfig, rng: np.random.Generator, std: float = 0.02, norm_jitter: float = 0.0):
    """Random-init frozen base with the shapes of include/tensor/base/frozen_base.hpp:31-56."""
    H, I, V = cfg.hidden, cfg.inter, cfg.vocab
    qd, kv = cfg.hq * cfg.hd, cfg.hkv * cfg.hd
    n = lambda *s: bf16_round(rng.standard_normal(s, dtype=F32) * F32(std))
    nw = lambda: bf16_round(np.ones(H, dtype=F32) + F32(norm_jitter) * rng.standard_normal(H, dtype=F32))
    base = {"embed": n(V, H), "final_norm": nw(), "layers": []}
    if not cfg.tie:
        base["lm_head"] = n(V, H)
    for _ in range(cfg.layers):
        base["layers"].append({
            "input_norm": nw(), "post_norm": nw(),
            "q_w": n(qd, H), "k_w": n(kv, H), "v_w": n(kv, H), "o_w": n(H, qd),
            "q_b": n(qd), "k_b": n(kv), "v_b": n(kv),
            "gate_w": n(I, H), "up_w": n(I, H), "down_w": n(H, I),
        })
    return base


def target_dims(cfg: BaseConfig, t: str) -> Tuple[int, int]:
    H, I = cfg.hidden, cfg.inter
    qd, kv = cfg.hq * cfg.hd, cfg.hkv * cfg.hd
    return {"q": (H, qd), "k": (H, kv), "v": (H, kv), "o": (qd, H),
            "gate": (H, I), "up": (H, I), "down": (I, H)}[t]


def make_adapter(cfg: BaseConfig, rank: int, targets=("q", "k", "v", "o"),
                 rng: Optional[np.random.Generator] = None, b_std: float = 0.0):
    """AdapterModel::create (src/adapter/adapter_model.cu:69-90): hash-Kaiming A, zero B. With an
    rng, B is drawn N(0, b_std) instead so that gA is not identically zero on the first step."""
    layers = []
    for _ in range(cfg.layers):
        la = {}
        for t in targets:
            i, o = target_dims(cfg, t)
            A = kaiming_init(i, rank)
            Bm = np.zeros((o, rank), dtype=F32) if rng is None else (rng.standard_normal((o, rank), dtype=F32) * F32(b_std))
            la[t] = LoraPair(A, Bm)
        layers.append(la)
    return layers


def qwen2_forward(cfg: BaseConfig, base, tokens: np.ndarray, B: int, T: int, adapter=None, scale: float = 1.0):
    """Qwen2Base::forward (src/base/arch/qwen2.cu:47-178), op for op, including the BF16 round after
    every GEMM / add and the LoRA delta added BEFORE RoPE (:104-111)."""
    H = cfg.hidden
    res = {"layer_cache": []}
    residual = embed_fwd(base["embed"], tokens)
    for l in range(cfg.layers):
        w = base["layers"][l]
        ad = adapter[l] if adapter is not None else {}
        lc = {"pre_attn_res": residual.copy()}
        lc["x_normed"], lc["in_rms"] = rms_norm_fwd(residual, w["input_norm"], cfg.eps)
        Q = add_bias(proj_fwd(w["q_w"], lc["x_normed"]), w["q_b"])
        K = add_bias(proj_fwd(w["k_w"], lc["x_normed"]), w["k_b"])
        V = add_bias(proj_fwd(w["v_w"], lc["x_normed"]), w["v_b"])
        if "q" in ad: Q = apply_lora_fwd(ad["q"], lc["x_normed"], Q, scale)
        if "k" in ad: K = apply_lora_fwd(ad["k"], lc["x_normed"], K, scale)
        if "v" in ad: V = apply_lora_fwd(ad["v"], lc["x_normed"], V, scale)
        Q = rope(Q, B, T, cfg.hq, cfg.hd, cfg.theta)
        K = rope(K, B, T, cfg.hkv, cfg.hd, cfg.theta)
        lc["Q"], lc["K"], lc["V"] = Q, K, V
        lc["attn_out"], lc["attn_w"] = sdpa_fwd(Q, K, V, B, T, cfg.hq, cfg.hkv, cfg.hd)
        h_mid = proj_fwd(w["o_w"], lc["attn_out"])
        if "o" in ad: h_mid = apply_lora_fwd(ad["o"], lc["attn_out"], h_mid, scale)
        residual = add_inplace(residual, h_mid)
        lc["pre_ffn_res"] = residual.copy()
        lc["x_normed2"], lc["post_rms"] = rms_norm_fwd(residual, w["post_norm"], cfg.eps)
        gate = proj_fwd(w["gate_w"], lc["x_normed2"])
        up = proj_fwd(w["up_w"], lc["x_normed2"])
        if "gate" in ad: gate = apply_lora_fwd(ad["gate"], lc["x_normed2"], gate, scale)
        if "up" in ad: up = apply_lora_fwd(ad["up"], lc["x_normed2"], up, scale)
        lc["gate_out"], lc["up_out"] = gate, up
        lc["act_out"] = silu_mul_fwd(gate, up)
        ffn = proj_fwd(w["down_w"], lc["act_out"])
        if "down" in ad: ffn = apply_lora_fwd(ad["down"], lc["act_out"], ffn, scale)
        residual = add_inplace(residual, ffn)
        res["layer_cache"].append(lc)
    res["x_final"] = residual.copy()
    xfn, res["final_rms"] = rms_norm_fwd(residual, base["final_norm"], cfg.eps)
    lm = base["embed"] if cfg.tie else base["lm_head"]
    res["logits"] = proj_fwd(lm, xfn)
    return res


def qwen2_backward(cfg: BaseConfig, base, fwd, dlogits: np.ndarray, B: int, T: int, adapter=None, scale: float = 1.0):
    """Qwen2Base::backward (src/base/arch/qwen2.cu:184-308). Returns per-layer dx_attn_in (the centroid
    gradient signal, :294-296); LoRA gradients accumulate into the adapter's gA/gB."""
    lm = base["embed"] if cfg.tie else base["lm_head"]
    dres = proj_bwd_x(lm, dlogits)
    grad = rms_norm_bwd(dres, fwd["x_final"], base["final_norm"], fwd["final_rms"])
    out = [None] * cfg.layers
    for l in range(cfg.layers - 1, -1, -1):
        w = base["layers"][l]; lc = fwd["layer_cache"][l]
        ad = adapter[l] if adapter is not None else {}
        dact = proj_bwd_x(w["down_w"], grad)
        if "down" in ad: dact = apply_lora_bwd(ad["down"], lc["act_out"], grad, dact, scale)
        dgate, dup = silu_mul_bwd(dact, lc["gate_out"], lc["up_out"])
        dxn2 = proj_bwd_x(w["gate_w"], dgate)
        dxn2 = proj_bwd_x(w["up_w"], dup, dxn2)
        if "gate" in ad: dxn2 = apply_lora_bwd(ad["gate"], lc["x_normed2"], dgate, dxn2, scale)
        if "up" in ad: dxn2 = apply_lora_bwd(ad["up"], lc["x_normed2"], dup, dxn2, scale)
        dffn_in = rms_norm_bwd(dxn2, lc["pre_ffn_res"], w["post_norm"], lc["post_rms"])
        grad = add_inplace(grad, dffn_in)
        dx_attn_out = proj_bwd_x(w["o_w"], grad)
        if "o" in ad: dx_attn_out = apply_lora_bwd(ad["o"], lc["attn_out"], grad, dx_attn_out, scale)
        dQ, dK, dV = sdpa_bwd(dx_attn_out, lc["Q"], lc["K"], lc["V"], lc["attn_w"], B, T, cfg.hq, cfg.hkv, cfg.hd)
        dQ = rope(dQ, B, T, cfg.hq, cfg.hd, cfg.theta, inverse=True)
        dK = rope(dK, B, T, cfg.hkv, cfg.hd, cfg.theta, inverse=True)
        dxn = proj_bwd_x(w["q_w"], dQ)
        dxn = proj_bwd_x(w["k_w"], dK, dxn)
        dxn = proj_bwd_x(w["v_w"], dV, dxn)
        if "q" in ad: dxn = apply_lora_bwd(ad["q"], lc["x_normed"], dQ, dxn, scale)
        if "k" in ad: dxn = apply_lora_bwd(ad["k"], lc["x_normed"], dK, dxn, scale)
        if "v" in ad: dxn = apply_lora_bwd(ad["v"], lc["x_normed"], dV, dxn, scale)
        out[l] = {"dx_attn_in": dxn.copy(), "dQ": dQ, "dK": dK, "dV": dV}
        dattn_in = rms_norm_bwd(dxn, lc["pre_attn_res"], w["input_norm"], lc["in_rms"])
        grad = add_inplace(grad, dattn_in)
    return out


# ───────────────────────────── optimiser / trainer host logic ─────────────────────────────

def adamw_step(master, m, v, grad, lr, b1, b2, eps, wd, step):
    """k_adamw (src/backend/cuda/ops.cu:1139-1158), in place; returns the BF16 working copy."""
    lr, b1, b2, eps, wd = map(F32, (lr, b1, b2, eps, wd))
    g = grad.astype(F32)
    m[...] = b1 * m + (F32(1) - b1) * g
    v[...] = b2 * v + (F32(1) - b2) * g * g
    bc1 = F32(1) - F32(np.power(b1, F32(step)))
    bc2 = F32(1) - F32(np.power(b2, F32(step)))
    mhat = m / bc1; vhat = v / bc2
    master[...] = master - lr * (mhat / (np.sqrt(vhat) + eps) + wd * master)
    return bf16_round(master)


def all_pairs(adapter) -> List[LoraPair]:
    return [lp for la in adapter for lp in la.values()]


def grad_norm(adapter) -> float:
    """compute_grad_norm (src/trainer/adapt_trainer.cu:32-44): sqrt of the FP32 sum of squares."""
    s = F32(0)
    for lp in all_pairs(adapter):
        s += np.sum(lp.gA * lp.gA, dtype=F32) + np.sum(lp.gB * lp.gB, dtype=F32)
    return float(np.sqrt(s))


def clip_gradients(adapter, max_norm: float, norm: float) -> None:
    """clip_gradients (src/trainer/adapt_trainer.cu:55-70): scale by max/(norm+1e-6) only if norm > max."""
    if norm <= max_norm:
        return
    s = F32(max_norm) / (F32(norm) + F32(1e-6))
    for lp in all_pairs(adapter):
        lp.gA *= s; lp.gB *= s


def adamw_step_all(adapter, lr, step, b1=0.9, b2=0.999, eps=1e-8, wd=0.0):
    """AdamW::step_all (src/trainer/adamw.cu:9-38)."""
    for lp in all_pairs(adapter):
        lp.A_bf16 = adamw_step(lp.A_f32, lp.mA, lp.vA, lp.gA, lr, b1, b2, eps, wd, step)
        lp.B_bf16 = adamw_step(lp.B_f32, lp.mB, lp.vB, lp.gB, lr, b1, b2, eps, wd, step)


def cosine_lr(base_lr: float, warmup: int, total: int, step: int, floor_frac: float = 0.1) -> float:
    """CosineSchedule::lr_at (include/tensor/trainer/cosine_schedule.hpp:18-29), FP32 arithmetic."""
    base_lr = F32(base_lr)
    if step < warmup:
        return float(base_lr * F32(step + 1) / F32(warmup))
    progress = F32(step - warmup) / F32(total - warmup)
    progress = min(progress, F32(1))
    cos_val = F32(0.5) * (F32(1) + F32(np.cos(F32(np.pi) * progress)))
    floor = base_lr * F32(floor_frac)
    return float(floor + (base_lr - floor) * cos_val)


IM_START, ASSISTANT, IM_END = 151644, 77091, 151645


def mask_targets(input_ids: np.ndarray, target_ids: np.ndarray, B: int, T: int) -> np.ndarray:
    """Assistant-only masking state machine (src/trainer/adapt_trainer.cu:145-182)."""
    tgt = target_ids.copy()
    for b in range(B):
        inside = False
        for t in range(T):
            i = b * T + t
            tok = int(input_ids[i])
            if tok == IM_START:
                inside = (t + 1 < T and int(input_ids[i + 1]) == ASSISTANT)
            mask = not inside
            if tok in (IM_START, ASSISTANT):
                mask = True
            if tok == IM_END:
                inside = False
                mask = False
            if mask:
                tgt[i] = -1
    return tgt


def mean_loss(loss_per_token: np.ndarray) -> float:
    """src/trainer/adapt_trainer.cu:237-246: FP32 running sum over entries > 1e-9, divided by their count."""
    s = F32(0); n = 0
    for l in loss_per_token.astype(F32):
        if l > F32(1e-9):
            s += l; n += 1
    return float(s / F32(n)) if n else 0.0


def next_batch(tokens: np.ndarray, pos: int, B: int, T: int):
    """Dataset::next_batch (src/data/dataset.cpp:55-71): sequential windows with wrap-around; targets
    are the next token. Returns (inputs, targets, new_pos)."""
    n = len(tokens)
    inp = np.empty(B * T, dtype=np.int32); tgt = np.empty(B * T, dtype=np.int32)
    for b in range(B):
        idx = (pos + np.arange(T)) % n
        inp[b * T:(b + 1) * T] = tokens[idx]
        tgt[b * T:(b + 1) * T] = tokens[(idx + 1) % n]
        pos = (pos + T) % n
    return inp, tgt, pos


# ───────────────────────────── centroid accumulator / merge ─────────────────────────────

_lib = None


def _kmeans_lib():
    global _lib
    if _lib is None:
        p = os.path.join(_HERE, "libkmeans_port.so")
        if not os.path.exists(p):
            raise RuntimeError("oracle/libkmeans_port.so is not built: run `make -C oracle port`")
        _lib = ctypes.CDLL(p)
        fp = ctypes.POINTER(ctypes.c_float); ip = ctypes.POINTER(ctypes.c_int)
        _lib.ta_oracle_kmeans.argtypes = [fp, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, fp, ip, ip]
        _lib.ta_oracle_kmeans.restype = ctypes.c_int
        _lib.ta_oracle_kmeans_from.argtypes = [fp, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ip, fp, ip]
        _lib.ta_oracle_kmeans_from.restype = ctypes.c_int
        for f in (_lib.ta_oracle_centroid_intended, _lib.ta_oracle_centroid_asbuilt):
            f.argtypes = [fp, fp, ctypes.c_int, ctypes.c_int, fp, fp]
            f.restype = None
    return _lib


def _fp(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def kmeans_merge(vectors: np.ndarray, k: int, max_iters: int = 50):
    """CentroidAccumulator::merge_and_write's k-means (src/centroid/centroid_accumulator.cpp:114-157)
    via oracle/kmeans_port.c. Returns (centers [k',D], assignments [N], passes executed)."""
    v = np.ascontiguousarray(vectors, dtype=F32)
    N, D = v.shape
    kk = min(k, N)
    centers = np.zeros((kk, D), dtype=F32)
    assign = np.zeros(N, dtype=np.int32)
    kout = ctypes.c_int(0)
    it = _kmeans_lib().ta_oracle_kmeans(_fp(v), N, D, k, max_iters, _fp(centers),
                                        assign.ctypes.data_as(ctypes.POINTER(ctypes.c_int)), ctypes.byref(kout))
    return centers, assign, it


class CentroidAccumulator:
    """Host state of include/tensor/centroid/centroid_accumulator.hpp:24-53: one FP32 accumulator of
    size D shared by all layers, never reset; snapshots are running means."""

    def __init__(self, D: int):
        self.D = D
        self.acc = np.zeros(D, dtype=F32)
        self.weight = np.zeros(1, dtype=F32)
        self.snapshots: List[np.ndarray] = []

    def accumulate(self, hidden: np.ndarray, grad: np.ndarray, mode: str = "intended"):
        h = np.ascontiguousarray(hidden, dtype=F32); g = np.ascontiguousarray(grad, dtype=F32)
        fn = _kmeans_lib().ta_oracle_centroid_intended if mode == "intended" else _kmeans_lib().ta_oracle_centroid_asbuilt
        fn(_fp(h), _fp(g), h.shape[0], h.shape[1], _fp(self.acc), _fp(self.weight))

    def snapshot(self) -> Optional[np.ndarray]:
        """write_snapshot (src/centroid/centroid_accumulator.cpp:72-91) without the file."""
        if self.weight[0] == 0:
            return None
        c = (self.acc / self.weight[0]).astype(F32)
        self.snapshots.append(c)
        return c


def write_snapshot_file(path: str, centroid: np.ndarray, weight: float) -> None:
    """Snapshot layout (src/centroid/centroid_accumulator.cpp:81-86): int32 D | D x f32 | f32 weight."""
    with open(path, "wb") as f:
        f.write(struct.pack("<i", len(centroid)))
        f.write(np.ascontiguousarray(centroid, dtype="<f4").tobytes())
        f.write(struct.pack("<f", weight))


def read_snapshot_file(path: str) -> Tuple[np.ndarray, float]:
    b = open(path, "rb").read()
    D = struct.unpack_from("<i", b, 0)[0]
    c = np.frombuffer(b, dtype="<f4", count=D, offset=4).copy()
    w = struct.unpack_from("<f", b, 4 + 4 * D)[0] if len(b) >= 8 + 4 * D else float("nan")
    return c, w


def write_merged_file(path: str, centers: np.ndarray) -> None:
    """Merged layout (src/centroid/centroid_accumulator.cpp:160-165): int32 k | int32 D | k*D f32."""
    k, D = centers.shape
    with open(path, "wb") as f:
        f.write(struct.pack("<ii", k, D))
        f.write(np.ascontiguousarray(centers, dtype="<f4").tobytes())


def read_merged_file(path: str) -> np.ndarray:
    b = open(path, "rb").read()
    k, D = struct.unpack_from("<ii", b, 0)
    return np.frombuffer(b, dtype="<f4", count=k * D, offset=8).reshape(k, D).copy()


def cfg1_vectors(seed: int = 0, n_snap: int = 32, per_snap: int = 64, D: int = 512, n_centres: int = 12,
                 sigma: float = 0.1):
    """Synthetic merge input (the 32 x 64 snapshot case): 12 Gaussian centres ~N(0,1), per-vector noise sigma=0.1,
    per-vector gradient mass lognormal(0,1). Returns (vectors [N,D] f32, mass [N] f32)."""
    rng = np.random.default_rng(seed)
    centres = rng.standard_normal((n_centres, D)).astype(F32)
    N = n_snap * per_snap
    which = rng.integers(0, n_centres, size=N)
    vec = (centres[which] + F32(sigma) * rng.standard_normal((N, D)).astype(F32)).astype(F32)
    mass = rng.lognormal(0.0, 1.0, size=N).astype(F32)
    return vec, mass


# Extensions with no reference implementation ("parity unpinned by the reference"): README.md:73-79
# promises seeded k-means++ initialisation and ranking of clusters by gradient mass.

def kmeans_pp_init(vectors: np.ndarray, k: int, seed: int) -> np.ndarray:
    """Seeded k-means++: first centre uniform, then proportional to squared distance (FP64 CDF).
    Uses a 64-bit LCG so the GPU build can reproduce the draws exactly. Returns chosen indices."""
    N = vectors.shape[0]
    state = (seed * 6364136223846793005 + 1442695040888963407) & (2 ** 64 - 1)

    def nxt():
        nonlocal state
        state = (state * 6364136223846793005 + 1442695040888963407) & (2 ** 64 - 1)
        return (state >> 11) / float(1 << 53)

    idx = [int(nxt() * N) % N]
    d2 = None
    for _ in range(1, k):
        diff = vectors - vectors[idx[-1]]
        nd = np.zeros(N, dtype=F32)
        # sequential FP32 sum over i, as the assignment distance
        for i in range(vectors.shape[1]):
            nd += diff[:, i] * diff[:, i]
        d2 = nd if d2 is None else np.minimum(d2, nd)
        cdf = np.cumsum(d2.astype(np.float64))
        r = nxt() * cdf[-1]
        idx.append(int(min(np.searchsorted(cdf, r, side="right"), N - 1)))
    return np.array(idx, dtype=np.int32)


def rank_by_mass(assign: np.ndarray, mass: np.ndarray, k: int) -> np.ndarray:
    """Cluster order by descending summed gradient mass (FP64 sums, stable for ties)."""
    tot = np.zeros(k, dtype=np.float64)
    np.add.at(tot, assign, mass.astype(np.float64))
    return np.argsort(-tot, kind="stable").astype(np.int32)


def kmeans_merge_ex(vectors: np.ndarray, mass: Optional[np.ndarray], k: int, seed: int, max_iters: int = 50):
    """Extension pipeline: seeded k-means++ start, the reference's Lloyd passes, clusters reordered by
    descending gradient mass. Returns (centers in ranked order, assignments in ranked labels, passes,
    ranked cluster masses, chosen start indices)."""
    v = np.ascontiguousarray(vectors, dtype=F32)
    N, D = v.shape
    kk = min(k, N)
    idx = kmeans_pp_init(v, kk, seed)
    centers = np.zeros((kk, D), dtype=F32)
    assign = np.zeros(N, dtype=np.int32)
    ip = ctypes.POINTER(ctypes.c_int)
    it = _kmeans_lib().ta_oracle_kmeans_from(_fp(v), N, D, kk, max_iters, idx.ctypes.data_as(ip), _fp(centers),
                                             assign.ctypes.data_as(ip))
    m = np.ones(N, dtype=F32) if mass is None else np.asarray(mass, dtype=F32)
    order = rank_by_mass(assign, m, kk)
    tot = np.zeros(kk, dtype=np.float64)
    np.add.at(tot, assign, m.astype(np.float64))
    inv = np.empty(kk, dtype=np.int32); inv[order] = np.arange(kk, dtype=np.int32)
    return centers[order], inv[assign], it, tot[order], idx


# Multi-vector snapshot banks (extension, no reference code): a snapshot FILE may hold several vectors, written as
# the reference's single-vector record (src/centroid/centroid_accumulator.cpp:81-86: int32 D | D x f32 | f32 weight)
# repeated back to back.  A one-record file is exactly the reference's snapshot; the reference's own reader sees the
# first record of a longer one.  The trainer's bank holds one gradient-weighted centroid per layer.

def write_bank_file(path: str, vectors: np.ndarray, weights: np.ndarray) -> None:
    with open(path, "wb") as f:
        for v, w in zip(np.asarray(vectors, dtype="<f4"), np.asarray(weights, dtype="<f4")):
            f.write(struct.pack("<i", len(v))); f.write(np.ascontiguousarray(v).tobytes()); f.write(struct.pack("<f", float(w)))


def read_bank_file(path: str) -> Tuple[np.ndarray, np.ndarray]:
    """All records of a snapshot file: (vectors [n, D], weights [n])."""
    b = open(path, "rb").read()
    vs, ws, off = [], [], 0
    while off + 4 <= len(b):
        D = struct.unpack_from("<i", b, off)[0]
        if D <= 0 or off + 8 + 4 * D > len(b):
            break
        vs.append(np.frombuffer(b, dtype="<f4", count=D, offset=off + 4).copy())
        ws.append(struct.unpack_from("<f", b, off + 4 + 4 * D)[0])
        off += 8 + 4 * D
    return np.array(vs, dtype=F32), np.array(ws, dtype=F32)


def layer_bank(hidden_per_layer, grad_per_layer) -> Tuple[np.ndarray, np.ndarray]:
    """One documented-formula centroid per layer: (acc_l / weight_l [L, D], weight_l [L])."""
    cs, ws = [], []
    for h, g in zip(hidden_per_layer, grad_per_layer):
        a = CentroidAccumulator(h.shape[1]); a.accumulate(h, g, "intended")
        cs.append((a.acc / a.weight[0]).astype(F32)); ws.append(a.weight[0])
    return np.array(cs, dtype=F32), np.array(ws, dtype=F32)


# ───────────────────────────── checkpoint files ─────────────────────────────

TARGET_NAMES = {"q": "self_attn.q_proj", "k": "self_attn.k_proj", "v": "self_attn.v_proj",
                "o": "self_attn.o_proj", "gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj"}


def safetensors_bytes(adapter) -> bytes:
    """write_f32_to_bf16_file (src/checkpoint/adapter_writer.cpp:30-72) + tensor order of
    write_safetensors (:74-91): u64 header length | JSON header (nlohmann `dump()`: keys sorted,
    no spaces) space-padded to a multiple of 8 | BF16 data in insertion order; each tensor is the
    RNE BF16 of the F32 master with a FLAT 1-D shape."""
    entries = {}
    data = bytearray()
    for l, la in enumerate(adapter):
        for t, lp in la.items():
            for suffix, arr in (("lora_A", lp.A_f32), ("lora_B", lp.B_f32)):
                b = bf16_bits(arr.reshape(-1)).astype("<u2").tobytes()
                name = f"layers.{l}.{TARGET_NAMES[t]}.{suffix}"
                entries[name] = {"data_offsets": [len(data), len(data) + len(b)], "dtype": "BF16",
                                 "shape": [arr.size]}
                data += b
    hdr = json.dumps(entries, sort_keys=True, separators=(",", ":"))
    while len(hdr) % 8:
        hdr += " "
    return struct.pack("<Q", len(hdr)) + hdr.encode() + bytes(data)


HF_LAYER_NAMES = {   # BaseLoader::load's tensor names (src/base/base_loader.cpp:112-160)
    "input_norm": "input_layernorm.weight", "post_norm": "post_attention_layernorm.weight",
    "q_w": "self_attn.q_proj.weight", "q_b": "self_attn.q_proj.bias", "k_w": "self_attn.k_proj.weight",
    "k_b": "self_attn.k_proj.bias", "v_w": "self_attn.v_proj.weight", "v_b": "self_attn.v_proj.bias",
    "o_w": "self_attn.o_proj.weight", "gate_w": "mlp.gate_proj.weight", "up_w": "mlp.up_proj.weight",
    "down_w": "mlp.down_proj.weight"}


def hf_tensor_dict(base) -> Dict[str, np.ndarray]:
    """The frozen base under the Hugging Face names BaseLoader::load asks for."""
    d = {"model.embed_tokens.weight": base["embed"], "model.norm.weight": base["final_norm"]}
    if "lm_head" in base:
        d["lm_head.weight"] = base["lm_head"]
    for l, lw in enumerate(base["layers"]):
        for k, name in HF_LAYER_NAMES.items():
            d[f"model.layers.{l}.{name}"] = lw[k]
    return d


def write_safetensors_file(path: str, tensors: Dict[str, np.ndarray], f32_names=(), metadata=None) -> None:
    """A safetensors file in the published layout (u64 LE header length | JSON | data): F32 arrays
    are stored as BF16 (their values must already be BF16-representable) unless named in f32_names."""
    hdr, data = {}, bytearray()
    if metadata:
        hdr["__metadata__"] = metadata
    for name, a in tensors.items():
        if name in f32_names:
            b, dt = np.ascontiguousarray(a, dtype="<f4").tobytes(), "F32"
        else:
            b, dt = bf16_bits(np.ascontiguousarray(a, dtype=F32).reshape(-1)).astype("<u2").tobytes(), "BF16"
        hdr[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [len(data), len(data) + len(b)]}
        data += b
    txt = json.dumps(hdr, separators=(",", ":"))
    while len(txt) % 8:
        txt += " "
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(txt)) + txt.encode() + bytes(data))


def write_hf_dir(d: str, cfg: "BaseConfig", base, shards: int = 1, f32_names=(), model_type: str = "qwen2") -> None:
    """config.json + model.safetensors (or model-0000i-of-0000n.safetensors shards, split round-robin)
    as BaseLoader::load / WeightMap::open expect them (src/parser/weight_map.cpp:26-68)."""
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump({"architectures": ["Qwen2ForCausalLM"], "model_type": model_type, "vocab_size": cfg.vocab,
                   "hidden_size": cfg.hidden, "num_hidden_layers": cfg.layers, "num_attention_heads": cfg.hq,
                   "num_key_value_heads": cfg.hkv, "intermediate_size": cfg.inter, "rms_norm_eps": cfg.eps,
                   "rope_theta": cfg.theta, "tie_word_embeddings": bool(cfg.tie), "torch_dtype": "bfloat16"}, f, indent=2)
    t = hf_tensor_dict(base)
    if shards == 1:
        write_safetensors_file(os.path.join(d, "model.safetensors"), t, f32_names, {"format": "pt"})
        return
    names = list(t)
    for i in range(shards):
        part = {n: t[n] for n in names[i::shards]}
        write_safetensors_file(os.path.join(d, f"model-{i + 1:05d}-of-{shards:05d}.safetensors"), part, f32_names, {"format": "pt"})


def base_sha(d: str) -> str:
    """sha256_dir (src/base/base_loader.cpp:30-52): SHA-256 of "name:size;" over the sorted *.safetensors."""
    import hashlib
    names = sorted(n for n in os.listdir(d) if n.endswith(".safetensors"))
    return hashlib.sha256("".join(f"{n}:{os.path.getsize(os.path.join(d, n))};" for n in names).encode()).hexdigest()


def _nlohmann_float(x: float) -> str:
    """nlohmann::json number_float dump: shortest round-trip of the double, '.0' appended when the
    text looks like an integer."""
    s = repr(float(x))
    if "e" in s or "E" in s:
        m, e = s.lower().split("e")
        s = f"{m}e{'-' if int(e) < 0 else '+'}{abs(int(e)):02d}"
    return s


def adapter_json_text(cfg: BaseConfig, rank: int, alpha: float, domain: str, step: int, tokens: int,
                      arch_name: str = "qwen2", base_sha: str = "synthetic",
                      inject: Optional[Dict[str, bool]] = None) -> str:
    """write_adapter_json (src/checkpoint/adapter_writer.cpp:93-128): nlohmann `dump(2)`, keys sorted."""
    inj = {"inject_q": True, "inject_k": True, "inject_v": True, "inject_o": True,
           "inject_up": False, "inject_down": False}
    if inject:
        inj.update(inject)
    j = {"domain": domain, "architecture": arch_name, "base_model": "unknown", "base_sha": base_sha,
         "rank": rank, "alpha": float(F32(alpha)), "target_begin": 0, "target_end": cfg.layers - 1,
         "tokens_trained": tokens, "centroid_dim": cfg.hidden, "centroid_count": 16, "step": step,
         "tensor_adapt_version": "0.1.0"}
    j.update(inj)
    lines = ["{"]
    keys = sorted(j)
    for i, k in enumerate(keys):
        v = j[k]
        if isinstance(v, bool):
            s = "true" if v else "false"
        elif isinstance(v, float):
            s = _nlohmann_float(v)
        elif isinstance(v, int):
            s = str(v)
        else:
            s = json.dumps(v, ensure_ascii=False)
        lines.append(f'  "{k}": {s}' + ("," if i + 1 < len(keys) else ""))
    lines.append("}")
    return "\n".join(lines)


def train_state_text(step: int, tokens: int) -> str:
    """src/checkpoint/adapter_writer.cpp:141-143."""
    return "{\n" + f'  "step": {step},\n  "tokens_consumed": {tokens}\n' + "}"


# ───────────────────────────── one full step ─────────────────────────────

def train_step(cfg: BaseConfig, base, adapter, tokens, targets, B, T, *, alpha, rank, lr, step,
               grad_clip=1.0, b1=0.9, b2=0.999, eps=1e-8, wd=0.0,
               centroid_intended: Optional[CentroidAccumulator] = None,
               centroid_asbuilt: Optional[CentroidAccumulator] = None):
    """Body of AdaptTrainer::Impl::do_step (src/trainer/adapt_trainer.cu:190-253) on given ids/targets."""
    scale = alpha / float(rank)
    for lp in all_pairs(adapter):
        lp.zero_grad()
    fwd = qwen2_forward(cfg, base, tokens, B, T, adapter, scale)
    loss, dlogits = cross_entropy_fwd(fwd["logits"], targets)
    lg = qwen2_backward(cfg, base, fwd, dlogits, B, T, adapter, scale)
    for l in range(cfg.layers):
        if centroid_intended is not None:
            centroid_intended.accumulate(fwd["layer_cache"][l]["x_normed"], lg[l]["dx_attn_in"], "intended")
        if centroid_asbuilt is not None:
            centroid_asbuilt.accumulate(fwd["layer_cache"][l]["x_normed"], lg[l]["dx_attn_in"], "asbuilt")
    grads = [(lp.gA.copy(), lp.gB.copy()) for lp in all_pairs(adapter)]
    norm = grad_norm(adapter)
    clip_gradients(adapter, grad_clip, norm)
    adamw_step_all(adapter, lr, step, b1, b2, eps, wd)
    return {"loss": loss, "mean_loss": mean_loss(loss), "grad_norm": norm, "grads": grads, "fwd": fwd, "layer_grads": lg}
