"""Data parallelism on real GPUs: a 2-rank NCCL run (torchrun, one process per GPU) of two optimiser
steps must give the single-GPU result on the same global batch - the LoRA gradients differ only by
FP32 reduction order, so masters agree to 1e-6 and the gradient norm to 1e-5 relative; the reported loss is the global-batch
mean and the job-wide centroid snapshot equals the single-GPU one.
Skipped when fewer than two GPUs are visible."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import refcase as rc

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_gpu_step_equals_single_gpu(ctx, tmp_path):
    from tensor_adapt_b200.trainer import AdaptTrainer, AdapterConfig
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "dp_worker.py")
    out = str(tmp_path / "dp.npz")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29731", worker, out],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stderr[-3000:]
    z = np.load(out)
    cfg = rc.tiny_cfg(hidden=256, hq=4, hkv=2, hd=64, inter=512)
    B, T, rank_r = 4, 128, 16
    base, adapter, toks, tgts = rc.make_case(cfg, B, T, rank_r, seed=21, steps=2, std=0.02, b_std=0.02)
    ac = AdapterConfig.defaults(rank=rank_r, alpha=32.0, targets=15, lr=2e-4, weight_decay=0.01, centroid_modes=1)
    tr = AdaptTrainer(ctx, rc.model_config(cfg), ac, B, T)
    rc.load_into_trainer(tr, cfg, base, adapter)
    for s in range(2):
        m = tr.step(toks[s], tgts[s], B, lr=2e-4)
        assert abs(m.grad_norm_raw - float(z[f"gnorm{s}"])) <= 1e-4 * m.grad_norm_raw
        assert abs(m.loss - float(z[f"loss{s}"])) <= 1e-5 * abs(m.loss)          # global-batch mean on every rank
        assert int(z[f"tokens{s}"]) == m.tokens_consumed == (s + 1) * B * T       # a rank counts the GLOBAL batch per step
        # Adam's sign-like first steps can flip on near-zero gradients: allow a few 2*lr outliers
        d = np.abs(tr.download("lora.master") - z[f"master{s}"])
        assert np.mean(d > 1e-6) < 1e-3 and d.max() <= 2.2 * 2e-4 * (s + 1)
    g = tr.download("lora.grad")
    assert rc.cosine(g, z["grad_last"]) >= 0.99999
    cen, w = tr.write_snapshot(2)
    assert abs(w - float(z["centroid_w"])) <= 1e-4 * w and float(z["local_w_after"].ravel()[0]) < 0.9 * w
    assert np.linalg.norm(cen - z["centroid"]) <= 1e-4 * np.linalg.norm(cen)
    tr.close()
