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
