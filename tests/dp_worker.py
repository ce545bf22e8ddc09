"""Worker for tests/test_gpu_dp.py: one rank of a data-parallel tiny training run (launched by torchrun)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
    sys.path.insert(0, p)
import refcase as rc  # noqa: E402
import tensor_adapt_b200 as ta  # noqa: E402
from tensor_adapt_b200.dp import Comm, DataParallelStep  # noqa: E402
from tensor_adapt_b200.trainer import AdaptTrainer, AdapterConfig  # noqa: E402


def main(out_path, exchange="torch"):
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = rc.tiny_cfg(hidden=256, hq=4, hkv=2, hd=64, inter=512)
    B, T, rank_r = 4, 128, 16
    base, adapter, toks, tgts = rc.make_case(cfg, B, T, rank_r, seed=21, steps=2, std=0.02, b_std=0.02)
    ctx = ta.Context(local)
    ac = AdapterConfig.defaults(rank=rank_r, alpha=32.0, targets=15, lr=2e-4, weight_decay=0.01, centroid_modes=1)
    tr = AdaptTrainer(ctx, rc.model_config(cfg), ac, B // world, T, stream=torch.cuda.current_stream().cuda_stream)
    rc.load_into_trainer(tr, cfg, base, adapter)
    comm = Comm(ctx, rank, world) if exchange == "library" else None      # C-level NCCL, per-layer overlapped buckets
    dp = DataParallelStep(tr, rank, world, comm=comm)
    out = {}
    for s in range(2):
        m = dp.step(toks[s], tgts[s], B, lr=2e-4)
        out[f"gnorm{s}"] = np.float32(m.grad_norm_raw)
        out[f"loss{s}"] = np.float32(m.loss)
        out[f"tokens{s}"] = np.int64(m.tokens_consumed)
        out[f"master{s}"] = tr.download("lora.master")
    out["grad_last"] = tr.download("lora.grad")
    out["centroid"], out["centroid_w"] = dp.write_snapshot(2)
    out["centroid_w"] = np.float32(out["centroid_w"])
    out["local_w_after"] = tr.download("centroid.weight")   # the rank's own sums survive the snapshot
    ctx.check_device()
    if rank == 0:
        np.savez(out_path, **out)
    dist.barrier()
    tr.close()
    if comm is not None:
        comm.close()
    ctx.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main(*sys.argv[1:3])
