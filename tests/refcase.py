"""Helpers shared by the parity tests and tests/golden/make_golden.py: seeded tiny models, the raw
case-directory format oracle/ref_harness.cu reads, and loading a model into the CUDA trainer."""
import os
import subprocess

import numpy as np

import ta_oracle as o

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HARNESS = os.path.join(ROOT, "oracle", "_ref", "ref_harness")
LAYER_KEYS = ["input_norm", "post_norm", "q_w", "k_w", "v_w", "o_w", "q_b", "k_b", "v_b", "gate_w", "up_w", "down_w"]


def tiny_cfg(**kw):
    d = dict(vocab=512, hidden=128, layers=2, hq=4, hkv=2, hd=64, inter=256, eps=1e-6, theta=1e6, tie=True)
    d.update(kw)
    return o.BaseConfig(**d)


def make_case(cfg, B, T, rank, targets=("q", "k", "v", "o"), seed=0, steps=1, std=0.05, b_std=0.05):
    """Seeded base, adapter (B != 0 so that gA is exercised on the first step) and token ids."""
    rng = np.random.default_rng(seed)
    base = o.make_base(cfg, rng, std=std, norm_jitter=0.1)
    adapter = o.make_adapter(cfg, rank, targets, rng=rng, b_std=b_std)
    toks, tgts = [], []
    for _ in range(steps):
        ids = rng.integers(0, cfg.vocab, size=B * T + 1).astype(np.int32)
        toks.append(ids[:-1].copy()); tgts.append(ids[1:].copy())
    return base, adapter, toks, tgts


def write_case_dir(d, cfg, base, adapter, toks, tgts, B, T, rank, alpha, **extra):
    """`base=None` leaves the weight files out: ref_harness then fills the base on the device with the same
    integer-hash generator as ta_trainer_init_random(seed 0), bit for bit."""
    os.makedirs(d, exist_ok=True)
    kv = dict(vocab=cfg.vocab, hidden=cfg.hidden, layers=cfg.layers, hq=cfg.hq, hkv=cfg.hkv, hd=cfg.hd, inter=cfg.inter,
              eps=cfg.eps, theta=cfg.theta, tie=int(cfg.tie), rank=rank, alpha=alpha, B=B, T=T, steps=len(toks))
    kv.update(extra)
    with open(os.path.join(d, "cfg.txt"), "w") as f:
        for k, v in kv.items():
            f.write(f"{k} {v}\n")
    w = lambda name, a: o.bf16_bits(a).astype("<u2").tofile(os.path.join(d, name + ".bin"))
    if base is not None:
        w("embed", base["embed"]); w("final_norm", base["final_norm"])
        if not cfg.tie:
            w("lm_head", base["lm_head"])
    for l in range(cfg.layers):
        if base is not None:
            for k in LAYER_KEYS:
                w(f"l{l}_{k}", base["layers"][l][k])
        for t, lp in adapter[l].items():
            lp.A_f32.astype("<f4").tofile(os.path.join(d, f"l{l}_lora_{t}_A.bin"))
            lp.B_f32.astype("<f4").tofile(os.path.join(d, f"l{l}_lora_{t}_B.bin"))
    for s, (a, b) in enumerate(zip(toks, tgts)):
        a.astype("<i4").tofile(os.path.join(d, f"tokens_{s}.bin")); b.astype("<i4").tofile(os.path.join(d, f"targets_{s}.bin"))


def run_harness(mode, case_dir, out_dir):
    r = subprocess.run([HARNESS, mode, case_dir, out_dir], capture_output=True, text=True, timeout=1800)
    if r.returncode != 0:
        raise RuntimeError(f"ref_harness {mode} failed: {r.stderr[-2000:]}")
    return r.stdout + r.stderr


def f32(path, shape=None):
    a = np.fromfile(path, dtype="<f4")
    return a.reshape(shape) if shape else a


def bf16(path, shape=None):
    a = o.bf16_from_bits(np.fromfile(path, dtype="<u2"))
    return a.reshape(shape) if shape else a


def load_into_trainer(tr, cfg, base, adapter):
    tr.upload("embed", base["embed"]); tr.upload("final_norm", base["final_norm"])
    if not cfg.tie:
        tr.upload("lm_head", base["lm_head"])
    for l, lw in enumerate(base["layers"]):
        for k in LAYER_KEYS:
            tr.upload(f"l{l}.{k}", lw[k])
        for t, lp in adapter[l].items():
            tr.upload(f"l{l}.lora.{t}.A", lp.A_f32); tr.upload(f"l{l}.lora.{t}.B", lp.B_f32)
    tr.sync_working()


def model_config(cfg):
    from tensor_adapt_b200.trainer import ModelConfig
    return ModelConfig(cfg.vocab, cfg.hidden, cfg.layers, cfg.hq, cfg.hkv, cfg.hd, cfg.inter, cfg.eps, cfg.theta, int(cfg.tie))


def cosine(a, b):
    a = np.asarray(a, np.float64).ravel(); b = np.asarray(b, np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300))


def relmax(a, b):
    return float(np.abs(np.asarray(a) - np.asarray(b)).max() / (np.abs(b).max() + 1e-30))


def hf_case(d, shards=2, seed=17):
    """Seeded Hugging Face style model directory (untied head, two F32 tensors whose values need rounding)
    shared by tests/golden/make_golden.py and the loader tests; returns (cfg, base)."""
    cfg = tiny_cfg(hidden=128, hq=2, hkv=1, hd=64, inter=256, vocab=320, layers=2)
    cfg.tie = False
    rng = np.random.default_rng(seed)
    base = o.make_base(cfg, rng, std=0.05, norm_jitter=0.1)
    base["layers"][1]["v_w"] = (rng.standard_normal(base["layers"][1]["v_w"].shape) * 0.05).astype(np.float32)
    base["lm_head"] = (rng.standard_normal(base["lm_head"].shape) * 0.05).astype(np.float32)
    o.write_hf_dir(d, cfg, base, shards=shards, f32_names={"model.layers.1.self_attn.v_proj.weight", "lm_head.weight"})
    return cfg, base
