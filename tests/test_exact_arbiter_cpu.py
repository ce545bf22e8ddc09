"""The exact-arithmetic arbiter (tests/exact_arbiter.py) against the pinned NumPy oracle on a tiny model, on the
CPU: same formulas (adjacent-pair RoPE, pre-RoPE LoRA delta, GQA causal attention, SwiGLU, cross-entropy scale,
both centroid accumulations), so the two may differ only by the oracle's BF16 rounding points."""
import numpy as np
import torch

import exact_arbiter as xa
import refcase as rc
import ta_oracle as o


def _case(targets, seed=5):
    cfg = rc.tiny_cfg(hidden=128, hq=4, hkv=2, hd=64, inter=256, vocab=512, layers=2)
    B, T, rank, alpha = 2, 64, 16, 32.0
    base, adapter, toks, tgts = rc.make_case(cfg, B, T, rank, targets=targets, seed=seed, std=0.05, b_std=0.05)
    return cfg, base, adapter, toks[0], tgts[0], B, T, rank, alpha


def test_exact_step_agrees_with_the_rounding_faithful_oracle():
    cfg, base, adapter, tok, tgt, B, T, rank, alpha = _case(("q", "k", "v", "o"))
    tgt = tgt.copy(); tgt[5:9] = -1                       # masked targets still carry gradient, as in the reference
    ex = xa.run_step(cfg, base, adapter, tok, tgt, B, T, alpha / rank, device="cpu")
    ci, ca = o.CentroidAccumulator(cfg.hidden), o.CentroidAccumulator(cfg.hidden)
    ref = o.train_step(cfg, base, adapter, tok, tgt, B, T, alpha=alpha, rank=rank, lr=0.0, step=1,
                       centroid_intended=ci, centroid_asbuilt=ca)
    assert abs(ex["loss"] - ref["mean_loss"]) <= 2e-3 * ref["mean_loss"]
    i = 0
    for l in range(cfg.layers):
        for t in ("q", "k", "v", "o"):
            gA, gB = ref["grads"][i]; i += 1
            assert xa.cosine(ex["grads"][(l, t)][0], gA) >= 0.999 and xa.cosine(ex["grads"][(l, t)][1], gB) >= 0.999
    for name, acc in (("intended", ci), ("asbuilt", ca)):
        a, w = ex["centroid"][name]
        assert abs(w - float(acc.weight[0])) <= 5e-3 * w
        assert xa.rel_l2(a / w, acc.acc / acc.weight[0]) <= 2e-2
    # the as-built accumulation only ever touches odd positions
    assert not ex["centroid"]["asbuilt"][0][0::2].any()


def test_rounding_emulation_moves_the_result_by_bf16_noise_only():
    """The emulation of the library's rounding points stays within BF16 noise of the exact step, and each
    rounding class changes the result (so switching one off attributes its share)."""
    cfg, base, adapter, tok, tgt, B, T, rank, alpha = _case(("q", "k", "v", "o", "gate", "up", "down"), seed=6)
    s = alpha / rank
    ex = xa.run_step(cfg, base, adapter, tok, tgt, B, T, s, device="cpu")
    em = xa.run_step(cfg, base, adapter, tok, tgt, B, T, s, rnd=xa.Rounding.library(), device="cpu")
    em32 = xa.run_step(cfg, base, adapter, tok, tgt, B, T, s, rnd=xa.Rounding.library_fp32_attention(), device="cpu")
    assert abs(em["loss"] - ex["loss"]) <= 2e-3 * ex["loss"]
    worst = max(xa.rel_l2(em["grads"][k][j], ex["grads"][k][j]) for k in ex["grads"] for j in (0, 1))
    worst32 = max(xa.rel_l2(em32["grads"][k][j], ex["grads"][k][j]) for k in ex["grads"] for j in (0, 1))
    assert 1e-4 < worst < 5e-2 and 1e-4 < worst32 < 5e-2
    assert any(not np.array_equal(em["grads"][k][0], em32["grads"][k][0]) for k in ex["grads"])
    # float32 evaluation of the exact graph is exact enough to arbitrate BF16-sized differences
    ex32 = xa.run_step(cfg, base, adapter, tok, tgt, B, T, s, device="cpu", dtype=torch.float32)
    assert max(xa.rel_l2(ex32["grads"][k][j], ex["grads"][k][j]) for k in ex["grads"] for j in (0, 1)) < 1e-4
