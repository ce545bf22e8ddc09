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


class DataParallelStep:
    """zero_grad -> local forward/backward on this rank's shard -> all-reduce -> optimiser step."""

    def __init__(self, trainer, rank: int, world: int):
        self.tr, self.rank, self.world = trainer, rank, world
        self.grad = trainer.torch_view("lora.grad")
        p, _, n, _, _ = trainer.tensor("centroid.weight")
        self._stats = None

    def step(self, tokens, targets, global_batch: int, lr: float = -1.0, total_steps: int = 0):
        tr = self.tr
        tok, tgt, b_local = shard_batch(tokens, targets, global_batch, tr.seq_len, self.rank, self.world)
        tr.zero_grad()
        tr.forward_backward(tok, tgt, b_local, global_tokens=global_batch * tr.seq_len)
        allreduce_sum_([self.grad])
        return tr.optimizer_step(lr, total_steps)
