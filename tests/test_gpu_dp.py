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
@pytest.mark.parametrize("exchange", ["torch", "library"])
def test_two_gpu_step_equals_single_gpu(ctx, tmp_path, exchange):
    """`torch`: one torch.distributed all-reduce of the flat gradient array; `library`: the C-level exchange
    (ta_comm_create + ta_trainer_set_comm), bucketed per layer and overlapped with the backward."""
    from tensor_adapt_b200.trainer import AdaptTrainer, AdapterConfig
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "dp_worker.py")
    out = str(tmp_path / "dp.npz")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29731" if exchange == "torch" else "29733", worker, out, exchange],
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


def test_library_exchange_with_one_rank_is_the_identity(ctx):
    """The C-level exchange on a single-rank communicator (runs on any box): per-layer buckets on the second stream
    and ta_allreduce_grads leave gradients, loss and the update exactly as the plain step produces them."""
    from tensor_adapt_b200.dp import Comm, DataParallelStep
    from tensor_adapt_b200.trainer import AdaptTrainer, AdapterConfig
    cfg = rc.tiny_cfg(hidden=256, hq=4, hkv=2, hd=64, inter=512, layers=3)
    B, T, rank_r = 4, 128, 16
    base, adapter, toks, tgts = rc.make_case(cfg, B, T, rank_r, seed=22, steps=2, std=0.02, b_std=0.02)
    ac = AdapterConfig.defaults(rank=rank_r, alpha=32.0, targets=127, lr=2e-4, weight_decay=0.01, centroid_modes=1)
    res = []
    for mode in ("plain", "attached", "explicit"):
        tr = AdaptTrainer(ctx, rc.model_config(cfg), ac, 2, T)          # two micro-batches per step
        rc.load_into_trainer(tr, cfg, base, adapter)
        comm = Comm(ctx, 0, 1) if mode != "plain" else None
        if mode == "attached":
            dp = DataParallelStep(tr, 0, 1, comm=comm)
            ms = [dp.step(toks[s], tgts[s], B, lr=2e-4) for s in range(2)]
        else:
            ms = []
            for s in range(2):
                tr.zero_grad(); tr.forward_backward(toks[s], tgts[s], B)
                if mode == "explicit":
                    tr._call("ta_allreduce_grads", comm.h)
                ms.append(tr.optimizer_step(2e-4))
        res.append((ms[-1].loss, ms[-1].grad_norm_raw, ms[-1].tokens_consumed, tr.download("lora.master"), tr.download("lora.grad")))
        ctx.check_device()
        tr.close()
        if comm:
            comm.close()
    for r in res[1:]:
        assert r[0] == res[0][0] and r[1] == res[0][1] and r[2] == res[0][2] == 2 * B * T
        np.testing.assert_array_equal(r[3], res[0][3]); np.testing.assert_array_equal(r[4], res[0][4])
