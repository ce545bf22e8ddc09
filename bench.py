#!/usr/bin/env python
"""Headline benchmark: LoRA training throughput of the B200-native step on Qwen2 shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config qwen2-7b]

One "step" is one optimiser step over the GLOBAL batch of the headline configuration (Qwen2-7B shapes, random
BF16 weights, LoRA r=16 alpha=32 on all seven projections, 32 sequences x 4096 uniform-random ids,
centroid accumulator on): zero_grad, forward, cross-entropy, backward, centroid accumulation,
grad-norm / clip / AdamW.  The global batch is fixed as N grows (strong scaling): each rank takes
32/N sequences, processes them in micro-batches and the flat LoRA gradient array is sum-reduced over
NCCL once per step.  Rank 0 prints ONE JSON line.

  value      tokens/s of the whole job with token ids already resident in HBM
  e2e        the same step through the public API with ids in pinned HOST memory (H2D inside the
             timed region) and the step metrics read back (D2H)
  roofline   the dominant kernel (segmented tcgen05 GEMM): algorithmic FLOPs of its launches / their
             summed CUDA-event time, measured in one extra profiled step, against the measured
             cuBLAS BF16 peak of this pool (MEASURED_PEAKS.json)
  cpu_baseline  the NumPy restatement of the reference (oracle/) timed on the host cores on a bounded
             sample of the same workload (rank 0, N=1 only)

`--impl reference` times the UNMODIFIED reference (its own CUDA build, oracle/_ref/ref_harness, the
reference has no CPU implementation of this path) on the same box at the largest micro-batch it can
run (its attention materialises FP32 [B,Hq,T,T] per layer and its loss kernel indexes with 32-bit
ints): LoRA on q/k/v/o only, no gradient accumulation.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # name: (model key, rank, alpha, targets, seq_len, global_batch, micro_batch)
    "qwen2-7b": ("qwen2-7b", 16, 32.0, 127, 4096, 32, 4),
    "qwen2-1.5b": ("qwen2-1.5b", 64, 128.0, 127, 2048, 16, 8),
    "qwen2-0.5b": ("qwen2-0.5b", 16, 32.0, 15, 1024, 8, 8),
}


# Model shapes as plain tuples (vocab, hidden, layers, q_heads, kv_heads, head_dim, intermediate, tied head):
# the reference arm and the CPU baseline read these, so neither has to load the CUDA library.
SHAPES = {
    "qwen2-0.5b": (151936, 896, 24, 14, 2, 64, 4864, 1),
    "qwen2-1.5b": (151936, 1536, 28, 12, 2, 128, 8960, 1),
    "qwen2-7b": (152064, 3584, 28, 28, 4, 128, 18944, 0),
}


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of the dominant kernel at the
# three most frequent shapes of the qwen2-7b step, from one ncu capture of
# `python -m tensor_adapt_b200.microbench gemm --M 16384 --N .. --K ..` (summary under profiles/), with the
# launches of each shape per layer pass; `roofline.traffic` is their launch-weighted mean.
NCU_GEMM_TRAFFIC_7B = {
    "16384x18944x3584 (gate, up, dX of down; CTA-pair kernel)": (1.308e9, 3),
    "16384x3584x18944 (down, halves of dX of gate+up; 256 x 224 single-CTA tiles)": (1.911e9, 3),
    "16384x3584x3584 (q, o and their dX; CTA-pair kernel)": (0.244e9, 4),
}


def flops_per_token(mc, rank, targets, T):
    """Algorithmic FLOPs per trained token: frozen base forward + dX (no base dW), causal attention at
    half-square, LoRA without recompute."""
    H, I, V, L = mc.hidden, mc.intermediate, mc.vocab, mc.layers
    qd, kv = mc.q_heads * mc.head_dim, mc.kv_heads * mc.head_dim
    p_lin = L * (H * qd + 2 * H * kv + qd * H + 3 * H * I)
    dims = [(H, qd), (H, kv), (H, kv), (qd, H), (H, I), (H, I), (I, H)]
    lora = sum(6 * rank * (i + o) * L for b, (i, o) in enumerate(dims) if targets & (1 << b))
    attn = 3.5 * L * (2 * T * qd)
    return 4 * (p_lin + V * H) + lora + attn


def measured_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))), "measured"
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.rows, self.p = gpu_index, [], None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.Q}",
                                       "--format=csv,noheader,nounits", "-lms", "200"],
                                      stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.p = None

    def _read(self):
        for line in self.p.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.p:
            self.p.terminate()
        sm = [float(r[1]) for r in self.rows if len(r) >= 8 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 8 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 8:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_baseline(cfg_name):
    """NumPy port of the reference step on ONE layer + lm head of the benchmark's shapes over 256
    tokens (T=256); tokens/s extrapolated as tokens / (L * t_layer + t_head)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import numpy as np
    import ta_oracle as o
    model, rank, alpha, targets, T, _, _ = CONFIGS[cfg_name]
    vocab, hidden, layers, hq, hkv, hd, inter, tie = SHAPES[model]
    T = 256
    cfg = o.BaseConfig(vocab=vocab, hidden=hidden, layers=1, hq=hq, hkv=hkv, hd=hd, inter=inter, tie=bool(tie))
    rng = np.random.default_rng(0)
    base = o.make_base(cfg, rng)
    tnames = [t for b, t in enumerate(o.ALL_TARGETS) if targets & (1 << b)]
    adapter = o.make_adapter(cfg, rank, tnames, rng=rng, b_std=0.02)
    ids = rng.integers(0, cfg.vocab, T + 1).astype(np.int32)
    scale = alpha / rank
    t0 = time.perf_counter()
    fwd = o.qwen2_forward(cfg, base, ids[:-1], 1, T, adapter, scale)
    t_head0 = time.perf_counter()
    loss, dlogits = o.cross_entropy_fwd(fwd["logits"], ids[1:])
    t1 = time.perf_counter()
    o.qwen2_backward(cfg, base, fwd, dlogits, 1, T, adapter, scale)
    t2 = time.perf_counter()
    # split head and layer cost: time the head products alone
    lm = base["embed"] if cfg.tie else base["lm_head"]
    th = time.perf_counter()
    o.proj_fwd(lm, fwd["x_final"]); o.proj_bwd_x(lm, dlogits)
    t_head = (time.perf_counter() - th) + (t1 - t_head0)
    t_layer = max((t2 - t0) - t_head, 1e-6)
    total = layers * t_layer + t_head
    try:
        import threadpoolctl
        cores = max([p.get("num_threads", 1) for p in threadpoolctl.threadpool_info()] + [1])
    except Exception:
        cores = os.cpu_count() or 1
    return {"value": T / total, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"NumPy restatement, 1 of {layers} layers + lm head of {model} shapes on {T} tokens "
                      f"(layer {t_layer:.2f}s, head {t_head:.2f}s), extrapolated to the full depth"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    model, lrank, alpha, _, T, _, _ = CONFIGS[args.config]
    vocab, hidden, layers, hq, hkv, hd, inter, tie = SHAPES[model]
    harness = os.path.join(ROOT, "oracle", "_ref", "ref_harness")
    base = {"impl": "reference", "metric": "lora_train_tokens_per_s", "unit": "tokens/s", "higher_is_better": True}
    if not os.path.exists(harness):
        print(json.dumps({**base, "unavailable": "oracle/_ref/ref_harness is not built (run make -C oracle on a box with the reference tree)"}))
        return
    # largest micro-batch the reference can hold: FP32 [B,Hq,T,T] per layer and int32 logit indexing
    B = {"qwen2-7b": 1, "qwen2-1.5b": 4, "qwen2-0.5b": 8}[args.config]
    d = tempfile.mkdtemp()
    with open(os.path.join(d, "cfg.txt"), "w") as f:
        f.write(f"vocab {vocab}\nhidden {hidden}\nlayers {layers}\nhq {hq}\nhkv {hkv}\n"
                f"hd {hd}\ninter {inter}\neps 1e-6\ntheta 1e6\ntie {tie}\n"
                f"rank {lrank}\nalpha {alpha}\nB {B}\nT {T}\nsteps {args.steps}\nwarmup_iters {args.warmup}\n"
                f"centroid 1\nlr 2e-4\nwd 0.01\n")
    t0 = time.time()
    r = subprocess.run([harness, "bench", d], capture_output=True, text=True)
    if r.returncode != 0:
        print(json.dumps({**base, "unavailable": "reference harness failed: " + r.stderr.strip().splitlines()[-1][:200]}))
        return
    j = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    v = j["tokens_per_s"]
    line = {**base, "value": v, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": j["ms_per_step"],
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{model} LoRA r{lrank} on q/k/v/o (the reference wires no other target), "
                                   f"{B} x {T} tokens per step, no gradient accumulation, centroid accumulator on; "
                                   "the reference's own CUDA build (it has no CPU implementation of this path)",
                       "largest_feasible": True, "global_batch": B, "seq_len": T, "targets": "q,k,v,o",
                       "why_not_the_headline_batch": "the reference materialises FP32 [B,Hq,T,T] per layer and indexes "
                                                     "logits with 32-bit ints, so larger micro-batches do not run; it has "
                                                     "no gradient accumulation, no gate/up/down adapters and no multi-GPU code",
                       "wall_s": round(time.time() - t0, 1)},
            "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": 1, "kind": "reference",
                             "sample": f"unmodified reference objects driven by oracle/ref_harness.cu, {B}x{T} tokens/step, "
                                       "one host thread + the GPU"},
            "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="qwen2-7b", choices=sorted(CONFIGS))
    ap.add_argument("--micro-batch", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", default="library", choices=["library", "torch"],
                    help="gradient exchange for N > 1: the library's per-layer NCCL buckets overlapped with the backward, "
                         "or one torch.distributed all-reduce after it")
    ap.add_argument("--cadence", type=int, default=0,
                    help="write a centroid snapshot and (rank 0) a checkpoint every this many steps inside the timed region")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import numpy as np
    import torch
    import torch.distributed as dist
    import tensor_adapt_b200 as ta
    from tensor_adapt_b200.dp import Comm, DataParallelStep, shard_batch
    from tensor_adapt_b200.trainer import QWEN2, AdaptTrainer, AdapterConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        # NCCL prints its version line on stdout when the communicator is created; stdout carries the one JSON
        # line only, so file descriptor 1 points at stderr while the process group comes up
        sys.stdout.flush()
        saved_fd = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_fd, 1)
            os.close(saved_fd)
    model, lrank, alpha, targets, T, gbatch, micro = CONFIGS[args.config]
    if args.micro_batch:
        micro = args.micro_batch
    mc = QWEN2[model]
    b_local = gbatch // world
    micro = min(micro, b_local)
    ctx = ta.Context(local)
    stream = torch.cuda.current_stream().cuda_stream
    ac = AdapterConfig.defaults(rank=lrank, alpha=alpha, targets=targets, lr=2e-4, weight_decay=0.01, centroid_modes=1)
    tr = AdaptTrainer(ctx, mc, ac, micro, T, stream=stream, output_dir=tempfile.mkdtemp() if args.cadence else None)
    tr.init_random(seed=1, std=0.02)
    # B != 0 so that every LoRA product does real work from the first step
    g = torch.Generator(device="cuda").manual_seed(7)
    tr.torch_view("lora.master").add_(torch.randn(tr.tensor("lora.master")[2], device="cuda", generator=g) * 0.01)
    tr.sync_working()
    grad = tr.torch_view("lora.grad")
    loss_stats = tr.torch_view("step.stats")[2:4]      # (sum of per-token losses, their count) of this rank's shard
    comm = None
    if world > 1 and args.exchange == "library":
        comm = Comm(ctx, rank, world)
        tr._call("ta_trainer_set_comm", comm.h)        # forward_backward now reduces each layer's slice as it completes

    gen = np.random.default_rng(1234)
    host_batches, dev_batches = [], []
    for s in range(2):   # two distinct global batches, alternated
        ids = gen.integers(0, mc.vocab, size=gbatch * T + 1).astype(np.int32)
        tok, tgt, _ = shard_batch(ids[:-1], ids[1:], gbatch, T, rank, world)
        ht, hg = torch.from_numpy(tok.copy()).pin_memory(), torch.from_numpy(tgt.copy()).pin_memory()
        host_batches.append((ht, hg)); dev_batches.append((ht.cuda(), hg.cuda()))
    global_tokens = gbatch * T

    def one_step(i, host):
        tok, tgt = (host_batches if host else dev_batches)[i & 1]
        tr.zero_grad()
        tr.forward_backward(tok, tgt, b_local, global_tokens=global_tokens)
        if world > 1 and comm is None:
            dist.all_reduce(grad)
            dist.all_reduce(loss_stats)                # so the reported loss is the global-batch mean on every rank
        m = tr.optimizer_step(2e-4)
        if args.cadence and m.step % args.cadence == 0:
            cadence_event(m.step)
        return m

    cadence_ms = []
    snapshotter = DataParallelStep(tr, rank, world, comm=comm)

    def cadence_event(step):
        """What AdaptTrainer does every checkpoint_every steps (src/trainer/adapt_trainer.cu:265-270): a centroid
        snapshot (sums reduced over the ranks first) and, on rank 0, the checkpoint files."""
        t0 = time.perf_counter()
        snapshotter.write_snapshot(step)               # sums of all ranks; rank 0 writes the file
        if rank == 0:
            tr.save_checkpoint(os.path.join(tr.output_dir, f"step-{step}"))
        cadence_ms.append((time.perf_counter() - t0) * 1e3)

    def timed(n, host):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            m = one_step(i, host)
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() / n, m

    for i in range(args.warmup):
        one_step(i, False)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    l0 = ctx.launches
    ms_dev, m = timed(args.steps, False)
    launches = (ctx.launches - l0) // max(args.steps, 1)
    ms_e2e, m2 = timed(args.steps, True)
    clocks = sampler.stop() if rank == 0 else None

    # one extra profiled step: CUDA-event time of every tensor-core launch by class
    import ctypes
    ctx.call("ta_profile_enable", 1)
    one_step(0, False)
    nl = (ctypes.c_long * 4)(); wk = (ctypes.c_double * 4)(); pm = (ctypes.c_double * 4)()
    ctx.call("ta_profile_read", 4, nl, wk, pm)
    ctx.call("ta_profile_enable", 0)
    ctx.check_device()

    if rank == 0:
        peaks, src = measured_peaks()
        fpt = flops_per_token(mc, lrank, targets, T)
        value = global_tokens / (ms_dev / 1e3)
        e2e = global_tokens / (ms_e2e / 1e3)
        gemm_tf = wk[0] / (pm[0] / 1e3) / 1e12 if pm[0] > 0 else None
        peak = peaks["bf16_tflops_sustained"]
        step_tf = fpt * global_tokens / world / (ms_dev / 1e3) / 1e12
        line = {
            "metric": "lora_train_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_dev, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "per_gpu_tokens_per_s": value / world,
            "config": {"workload": f"{model} shapes, random-init BF16 base, LoRA r{lrank} alpha {alpha:g} on "
                                   f"{bin(targets).count('1')} projections, global batch {gbatch} x {T} tokens, "
                                   f"micro-batch {micro} sequences, AdamW + grad clip + centroid accumulator",
                       "global_batch": gbatch, "seq_len": T, "micro_batch": micro, "parallelism": f"dp{world}",
                       "exchange": ("none" if world == 1 else "library: per-layer NCCL all-reduce buckets on a second stream, "
                                    "overlapped with the backward" if comm is not None else "torch.distributed all-reduce after the backward"),
                       "cadence": ({"every_steps": args.cadence, "events_in_timed_regions": len(cadence_ms),
                                    "ms_per_event": (sum(cadence_ms) / len(cadence_ms)) if cadence_ms else None,
                                    "what": "centroid snapshot + rank-0 checkpoint (adapter.safetensors, adapter.json, "
                                            "train_state.json, optimizer.safetensors)"} if args.cadence else None),
                       "l2": "per-step working set (>=15 GB of weights + activations) far exceeds the 126 MB L2; no flush needed",
                       "loss": m.loss, "grad_norm": m.grad_norm_raw},
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": 2 * 4 * b_local * T * world, "d2h_bytes_per_step": 16 * world},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "achieved": gemm_tf, "peak": peak, "unit": "TFLOP/s",
                         "frac": (gemm_tf / peak) if gemm_tf else None,
                         "traffic": (sum(b * n for b, n in NCU_GEMM_TRAFFIC_7B.values()) / sum(n for _, n in NCU_GEMM_TRAFFIC_7B.values())
                                     if args.config == "qwen2-7b" else None),
                         "traffic_note": ("bytes per launch, launch-weighted mean of ncu captures of the three dominant shapes; "
                                          "algorithmic operand + output bytes of the same mix: 0.63e9" if args.config == "qwen2-7b" else None),
                         "peak_source": f"{src} bf16_tflops_sustained (kernel timed inside a long step)",
                         "kernel": "seg_gemm_kernel + seg_gemm_pair3_kernel (tiles >= 128 wide)", "kernel_launches": int(nl[0]),
                         "kernel_ms_per_step": pm[0], "kernel_share_of_step": pm[0] / ms_dev,
                         "step_tflops_per_gpu": step_tf, "step_frac_of_burst_peak": step_tf / peaks["bf16_tflops"],
                         "step_frac_of_sustained_peak": step_tf / peak,
                         "flops_per_token": fpt,
                         "other_ms_per_step": {"skinny_gemm": pm[1], "attention_fwd": pm[2], "attention_bwd": pm[3]},
                         "attention_tflops": {"fwd": wk[2] / (pm[2] / 1e3) / 1e12 if pm[2] else None,
                                              "bwd": wk[3] / (pm[3] / 1e3) / 1e12 if pm[3] else None}},
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            try:
                line["cpu_baseline"] = cpu_baseline(args.config)
            except Exception as e:   # the baseline is a report, never a reason to lose the bench line
                line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
        print(json.dumps(line))
    tr.close()
    if comm is not None:
        comm.close()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
