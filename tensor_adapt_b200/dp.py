"""Data-parallel plumbing: one process per GPU, torch.distributed for the only exchange of the step.

Sequences are independent, so the global batch is sharded by sequence with no data-path collective;
the frozen base and the LoRA state are replicated.  Once per optimiser step the flat FP32 LoRA
gradient array is sum-reduced (each rank already scaled its cross-entropy gradient by
1/global_tokens, so the sum is the global-batch gradient the single-GPU step computes) together with
the loss numerator / count; grad-norm, clip and AdamW then run identically on every rank.  Centroid
accumulators are sums and are reduced only when a snapshot is written.
"""
from __future__ import annotations


def shard_range(global_batch: int, rank: int, world: int):
    """Sequences [lo, hi) of the global batch owned by `rank` (equal shards required)."""
    if global_batch % world:
        raise ValueError(f"global batch {global_batch} is not divisible by world size {world}")
    per = global_batch // world
    return rank * per, (rank + 1) * per


def shard_batch(tokens, targets, global_batch: int, seq_len: int, rank: int, world: int):
    lo, hi = shard_range(global_batch, rank, world)
    return tokens[lo * seq_len:hi * seq_len], targets[lo * seq_len:hi * seq_len], hi - lo


def allreduce_sum_(tensors, group=None):
    """In-place SUM all-reduce of each tensor (torch tensors on the backend's device)."""
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    for t in tensors:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)


class Comm:
    """NCCL communicator owned by the C library (ta_comm_*): rank 0 draws the unique id, the bytes travel to the
    other ranks over the already-initialised torch.distributed group (any backend; gloo is enough)."""

    def __init__(self, ctx, rank: int, world: int, group=None):
        import ctypes
        import torch
        import torch.distributed as dist
        from ._lib import lib, TAError
        buf = (ctypes.c_ubyte * 128)()
        if rank == 0:
            rc = lib.ta_comm_unique_id(buf, 128)
            if rc:
                raise TAError(rc, "ta_comm_unique_id (is NCCL loadable?)")
        if world > 1:
            t = torch.tensor(list(buf), dtype=torch.uint8)
            if dist.get_backend(group) == "nccl":
                t = t.cuda()
            dist.broadcast(t, src=0, group=group)
            buf = (ctypes.c_ubyte * 128)(*t.cpu().tolist())
        h = ctypes.c_void_p()
        ctx.call("ta_comm_create", rank, world, buf, 128, ctypes.byref(h))
        self.h, self.ctx, self.rank, self.world = h, ctx, rank, world

    def close(self):
        if self.h:
            from ._lib import lib
            lib.ta_comm_destroy(self.h)
            self.h = None


class DataParallelStep:
    """zero_grad -> local forward/backward on this rank's shard -> all-reduce -> optimiser step.

    Reduced per step: the flat LoRA gradient array and the (loss sum, loss count) pair, so every rank
    reports the global-batch mean loss of src/trainer/adapt_trainer.cu:237-246.  Reduced per snapshot:
    the centroid sums (`write_snapshot`); each rank keeps its own running sums in between."""

    def __init__(self, trainer, rank: int, world: int, group=None, comm: "Comm | None" = None):
        """With `comm` the exchange runs inside the library: per-layer buckets all-reduced on a second stream while
        the backward of the remaining layers proceeds (ta_trainer_set_comm); without it, one torch all-reduce."""
        self.tr, self.rank, self.world, self.group, self.comm = trainer, rank, world, group, comm
        self.grad = trainer.torch_view("lora.grad")
        self.stats = trainer.torch_view("step.stats")
        if comm is not None:
            trainer._call("ta_trainer_set_comm", comm.h)

    def step(self, tokens, targets, global_batch: int, lr: float = -1.0, total_steps: int = 0):
        tr = self.tr
        tok, tgt, b_local = shard_batch(tokens, targets, global_batch, tr.seq_len, self.rank, self.world)
        tr.zero_grad()
        tr.forward_backward(tok, tgt, b_local, global_tokens=global_batch * tr.seq_len)
        if self.comm is None:
            allreduce_sum_([self.grad, self.stats[2:4]], self.group)
        return tr.optimizer_step(lr, total_steps)

    def write_snapshot(self, step: int, mode: int = 0):
        """CentroidAccumulator::write_snapshot (src/centroid/centroid_accumulator.cpp:72-91) over the
        whole job: the per-rank sums are added (sums commute), every rank normalises the same global
        centroid and keeps it for the final merge, only rank 0 writes the file."""
        tr = self.tr
        names = ("centroid.acc", "centroid.weight") if mode == 0 else ("centroid_asbuilt.acc", "centroid_asbuilt.weight")
        views = [tr.torch_view(n) for n in names]
        local = [v.clone() for v in views]
        allreduce_sum_(views, self.group)
        out_dir = tr.output_dir
        if self.rank != 0:
            tr.output_dir = None
        try:
            return tr.write_snapshot(step, mode)
        finally:
            tr.output_dir = out_dir
            for v, l in zip(views, local):
                v.copy_(l)
