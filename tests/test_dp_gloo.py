"""Data-parallel semantics with two CPU ranks over gloo: sharding the global batch by sequence,
scaling each rank's cross-entropy gradient by 1/global_tokens and SUM-reducing the LoRA gradients
(tensor_adapt_b200.dp) reproduces the single-process global-batch gradients, loss sums and centroid
sums.  The per-rank compute is the NumPy oracle (no GPU here); the GPU path uses the same helpers."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank_main(rank, world, port, out_dir):
    for p in (ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
        sys.path.insert(0, p)
    import refcase as rc
    import ta_oracle as o
    from tensor_adapt_b200.dp import allreduce_sum_, shard_batch
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = rc.tiny_cfg(hidden=128, hq=2, hkv=1, hd=64, inter=256, vocab=256, layers=1)
    B, T, r = 4, 32, 16
    base, adapter, toks, tgts = rc.make_case(cfg, B, T, r, seed=5, std=0.02, b_std=0.02)
    tok, tgt, b_local = shard_batch(toks[0], tgts[0], B, T, rank, world)
    fwd = o.qwen2_forward(cfg, base, tok, b_local, T, adapter, 2.0)
    loss, dlogits = o.cross_entropy_fwd(fwd["logits"], tgt)
    dlogits = dlogits * np.float32(b_local * T / (B * T))     # 1/local -> 1/global (a power of two: exact)
    lg = o.qwen2_backward(cfg, base, fwd, dlogits, b_local, T, adapter, 2.0)
    cen = o.CentroidAccumulator(cfg.hidden)
    cen.accumulate(fwd["layer_cache"][0]["x_normed"], lg[0]["dx_attn_in"])
    flat = torch.from_numpy(np.concatenate([np.concatenate([lp.gA.ravel(), lp.gB.ravel()]) for lp in o.all_pairs(adapter)]))
    stats = torch.tensor([float(loss.sum()), float(len(loss))], dtype=torch.float64)
    cen_t = torch.from_numpy(np.concatenate([cen.acc, cen.weight]).astype(np.float64))
    allreduce_sum_([flat, stats, cen_t])
    if rank == 0:
        np.savez(os.path.join(out_dir, "dp.npz"), flat=flat.numpy(), stats=stats.numpy(), cen=cen_t.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_data_parallel_equals_single_process(tmp_path):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import refcase as rc
    import ta_oracle as o
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    z = np.load(tmp_path / "dp.npz")
    cfg = rc.tiny_cfg(hidden=128, hq=2, hkv=1, hd=64, inter=256, vocab=256, layers=1)
    B, T, r = 4, 32, 16
    base, adapter, toks, tgts = rc.make_case(cfg, B, T, r, seed=5, std=0.02, b_std=0.02)
    fwd = o.qwen2_forward(cfg, base, toks[0], B, T, adapter, 2.0)
    loss, dlogits = o.cross_entropy_fwd(fwd["logits"], tgts[0])
    lg = o.qwen2_backward(cfg, base, fwd, dlogits, B, T, adapter, 2.0)
    cen = o.CentroidAccumulator(cfg.hidden)
    cen.accumulate(fwd["layer_cache"][0]["x_normed"], lg[0]["dx_attn_in"])
    flat = np.concatenate([np.concatenate([lp.gA.ravel(), lp.gB.ravel()]) for lp in o.all_pairs(adapter)])
    # sequences are independent, so only FP32 summation order differs
    assert rc.cosine(z["flat"], flat) >= 0.999999 and rc.relmax(z["flat"], flat) <= 1e-3
    assert abs(z["stats"][0] - float(loss.sum())) <= 1e-4 * float(loss.sum()) and z["stats"][1] == B * T
    ref_c = np.concatenate([cen.acc, cen.weight])
    assert np.abs(z["cen"] - ref_c).max() <= 1e-3 * np.abs(ref_c).max()


class _FakeTrainer:
    """Host-side stand-in with the attributes DataParallelStep touches (CPU tensors instead of HBM)."""

    def __init__(self, rank, out_dir):
        self.seq_len, self.rank, self.output_dir = 4, rank, out_dir
        self.t = {"lora.grad": torch.zeros(6), "step.stats": torch.zeros(4), "centroid.acc": torch.zeros(3),
                  "centroid.weight": torch.zeros(1)}
        self.written = []
        self.tokens_consumed = 0
        self.pending = 0

    def torch_view(self, name):
        return self.t[name]

    def zero_grad(self):
        self.t["lora.grad"].zero_(); self.t["step.stats"].zero_()

    def forward_backward(self, tok, tgt, b_local, global_tokens=0):
        self.t["lora.grad"] += float(np.sum(tok)) / global_tokens
        self.pending = global_tokens          # the library counts the step's GLOBAL tokens once, on every rank
        self.t["step.stats"][2] += float(np.sum(tgt)); self.t["step.stats"][3] += len(tgt)
        self.t["centroid.acc"] += self.rank + 1.0; self.t["centroid.weight"] += 2.0

    def optimizer_step(self, lr, total_steps):
        s = self.t["step.stats"]
        self.tokens_consumed += self.pending; self.pending = 0
        return float(s[2] / s[3]), self.t["lora.grad"].clone()

    def write_snapshot(self, step, mode=0):
        self.written.append(self.output_dir)
        return (self.t["centroid.acc"] / self.t["centroid.weight"]).numpy().copy(), float(self.t["centroid.weight"])


def _dp_step_main(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    from tensor_adapt_b200.dp import DataParallelStep
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    tr = _FakeTrainer(rank, out_dir)
    dp = DataParallelStep(tr, rank, world)
    toks = np.arange(16, dtype=np.int32); tgts = np.arange(16, dtype=np.int32) * 2
    loss, grad = dp.step(toks, tgts, global_batch=4)
    cen, w = dp.write_snapshot(1)
    np.savez(os.path.join(out_dir, f"r{rank}.npz"), loss=loss, grad=grad.numpy(), cen=cen, w=w,
             local_w=tr.t["centroid.weight"].numpy(), tokens=np.int64(tr.tokens_consumed), wrote=np.array([d is not None for d in tr.written]),
             out_dir_kept=np.array(tr.output_dir == out_dir))
    dist.barrier()
    dist.destroy_process_group()


def test_data_parallel_step_reduces_grads_loss_and_snapshot(tmp_path):
    port = 31500 + (os.getpid() % 2000)
    mp.spawn(_dp_step_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    z0, z1 = np.load(tmp_path / "r0.npz"), np.load(tmp_path / "r1.npz")
    for z in (z0, z1):
        assert float(z["loss"]) == pytest.approx(np.arange(16).sum() * 2 / 16)      # global mean on every rank
        np.testing.assert_allclose(z["grad"], np.full(6, np.arange(16).sum() / 16.0), rtol=1e-6)
        np.testing.assert_allclose(z["cen"], np.full(3, 3.0 / 4.0))                  # (1 + 2) / (2 + 2)
        assert float(z["w"]) == 4.0 and float(z["local_w"][0]) == 2.0                # local sums restored
        assert bool(z["out_dir_kept"])
        assert int(z["tokens"]) == 16                                               # global batch 4 x seq_len 4, not the shard
    assert z0["wrote"].tolist() == [True] and z1["wrote"].tolist() == [False]        # only rank 0 gets a path
