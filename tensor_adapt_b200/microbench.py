"""Per-kernel timing of the library's entry points with CUDA events (also the small cases profiled
with ncu; the summaries under profiles/ name the exact command lines).

    python -m tensor_adapt_b200.microbench attention --B 1 --T 4096 --Hq 28 --Hkv 4 --hd 128
    python -m tensor_adapt_b200.microbench gemm --M 16384 --N 3584 --K 3584 [--b-layout 1]
    python -m tensor_adapt_b200.microbench rowops --rows 16384 --D 3584 --I 18944
    python -m tensor_adapt_b200.microbench lora --BT 4096 --in 896 --out 896 --rank 16
    python -m tensor_adapt_b200.microbench skinny --BT 16384 --in 3584 --out 18944 --rank 16
    python -m tensor_adapt_b200.microbench kmeans --N 2048 --D 512 --k 8

Each line reports the median of `--iters` launches after `--warmup`; inputs are larger than L2 or the
L2 is flushed between launches (a 256 MB buffer is rewritten) when `--flush` is given.
"""
import argparse
import json
import statistics

import torch

import tensor_adapt_b200 as ta
from tensor_adapt_b200 import ptr, stream_ptr

HBM_PEAK = None


def timeit(fn, iters, warmup, flush):
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        if flush:
            scratch.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return statistics.median(ts)


def rnd(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def report(name, ms, flops=None, bytes_=None, **kw):
    d = {"kernel": name, "ms": round(ms, 4)}
    if flops:
        d["tflops"] = round(flops / ms / 1e9, 1)
    if bytes_:
        d["gb_per_s"] = round(bytes_ / ms / 1e6, 1)
    d.update(kw)
    print(json.dumps(d))


def attention(ctx, a):
    B, T, Hq, Hkv, hd = a.B, a.T, a.Hq, a.Hkv, a.hd
    Q, K, V, dO = rnd(B * T, Hq * hd), rnd(B * T, Hkv * hd), rnd(B * T, Hkv * hd), rnd(B * T, Hq * hd)
    out = torch.empty_like(Q); lse = torch.empty(B * Hq * T, device="cuda")
    dQ, dK, dV = torch.empty_like(Q), torch.empty_like(K), torch.empty_like(V)
    delta = torch.empty(B * Hq * T, device="cuda")
    pair = 2.0 * B * Hq * T * T * hd * 0.5   # one causal contraction
    f = lambda: ctx.call("ta_flash_attn_fwd", ptr(Q), ptr(K), ptr(V), ptr(out), ptr(lse), B, T, Hq, Hkv, hd, stream_ptr())
    b = lambda: ctx.call("ta_flash_attn_bwd", ptr(dO), ptr(Q), ptr(K), ptr(V), ptr(out), ptr(lse), ptr(dQ), ptr(dK), ptr(dV),
                         ptr(delta), B, T, Hq, Hkv, hd, stream_ptr())
    report("flash_attn_fwd", timeit(f, a.iters, a.warmup, a.flush), flops=2 * pair, shape=[B, T, Hq, Hkv, hd])
    report("flash_attn_bwd", timeit(b, a.iters, a.warmup, a.flush), flops=5 * pair, shape=[B, T, Hq, Hkv, hd],
           note="5 contractions counted, 7 executed")


def gemm(ctx, a):
    M, N, K = a.M, a.N, a.K
    A = rnd(M, K); Bm = rnd(K, N) if a.b_layout else rnd(N, K)
    C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    f = lambda: ctx.call("ta_gemm_bf16", M, N, K, 1.0, ptr(A), K, 0, ptr(Bm), Bm.shape[1], a.b_layout, None, None, ptr(C), N,
                         stream_ptr())
    if a.tile or a.pair:
        bn, mh = (int(v) for v in a.tile.split(",")) if a.tile else (0, 0)
        ctx.call("ta_ctx_set_gemm_tuning", bn, mh, a.pair)
    if a.raster:
        gm, gn = (int(v) for v in a.raster.split(","))
        ctx.call("ta_ctx_set_gemm_raster", gm, gn)
    report("gemm_bf16", timeit(f, a.iters, a.warmup, a.flush), flops=2.0 * M * N * K, shape=[M, N, K], b_layout=a.b_layout,
           tile=a.tile or "auto", pair=a.pair, raster=a.raster or "default")
    ctx.call("ta_ctx_set_gemm_tuning", 0, 0, 0)
    ctx.call("ta_ctx_set_gemm_raster", 0, 0)


def lora(ctx, a):
    BT, ind, od, r = a.BT, getattr(a, "in"), a.out, a.rank
    x, W, dY = rnd(BT, ind), rnd(od, ind, scale=0.02), rnd(BT, od)
    A, Bm = rnd(r, ind, scale=0.03), rnd(od, r, scale=0.02)
    y = torch.empty(BT, od, device="cuda", dtype=torch.bfloat16); dX = torch.empty(BT, ind, device="cuda", dtype=torch.bfloat16)
    gA = torch.zeros(r, ind, device="cuda"); gB = torch.zeros(od, r, device="cuda")
    f = lambda: ctx.call("ta_lora_linear_fwd", ptr(x), ptr(W), None, ptr(A), ptr(Bm), None, ptr(y), BT, ind, od, r, 2.0, stream_ptr())
    b = lambda: ctx.call("ta_lora_linear_bwd", ptr(x), ptr(dY), ptr(W), ptr(A), ptr(Bm), ptr(dX), 0, ptr(gA), ptr(gB), BT, ind, od,
                         r, 2.0, stream_ptr())
    ff = 2.0 * BT * (ind * od + r * (ind + od))
    report("lora_linear_fwd", timeit(f, a.iters, a.warmup, a.flush), flops=ff, shape=[BT, ind, od, r])
    report("lora_linear_bwd", timeit(b, a.iters, a.warmup, a.flush), flops=2.0 * BT * (ind * od + 3 * r * (ind + od)),
           shape=[BT, ind, od, r])


def skinny(ctx, a):
    """The four rank-r products of one adapted projection, each HBM-bound: bytes = the big operand once."""
    BT, ind, od, r = a.BT, getattr(a, "in"), a.out, a.rank
    x, dY = rnd(BT, ind), rnd(BT, od)
    A, Bm = rnd(r, ind, scale=0.03), rnd(od, r, scale=0.02)
    h = torch.empty(BT, r, device="cuda", dtype=torch.bfloat16); dh = torch.empty_like(h)
    gA = torch.zeros(r, ind, device="cuda"); gB = torch.zeros(od, r, device="cuda")
    t = timeit(lambda: ctx.call("ta_gemm_bf16", BT, r, ind, 2.0, ptr(x), ind, 0, ptr(A), ind, 0, None, None, ptr(h), r, stream_ptr()),
               a.iters, a.warmup, a.flush)
    report("h = x.A^T", t, bytes_=2.0 * BT * ind, shape=[BT, ind, r])
    t = timeit(lambda: ctx.call("ta_gemm_bf16", BT, r, od, 2.0, ptr(dY), od, 0, ptr(Bm), r, 1, None, None, ptr(dh), r, stream_ptr()),
               a.iters, a.warmup, a.flush)
    report("dh = dY.B", t, bytes_=2.0 * BT * od, shape=[BT, od, r])
    t = timeit(lambda: ctx.call("ta_gemm_tokens_f32", od, r, BT, 1.0, ptr(dY), od, ptr(h), r, ptr(gB), r, 1, 0, stream_ptr()),
               a.iters, a.warmup, a.flush)
    report("gB += dY^T.h", t, bytes_=2.0 * BT * (od + r), shape=[od, r, BT])
    t = timeit(lambda: ctx.call("ta_gemm_tokens_f32", ind, r, BT, 1.0, ptr(x), ind, ptr(dh), r, ptr(gA), ind, 1, 1, stream_ptr()),
               a.iters, a.warmup, a.flush)
    report("gA += dh^T.x", t, bytes_=2.0 * BT * (ind + r), shape=[ind, r, BT])


def swiglu(ctx, a):
    """The MLP's gate/up projection + SwiGLU and the down projection's dX + SwiGLU backward: separate kernels
    against the launches that fold SwiGLU into the GEMM epilogue."""
    BT, H, I = a.rows, a.D, a.I
    x, Wg, Wu, Wd = rnd(BT, H), rnd(I, H, scale=0.02), rnd(I, H, scale=0.02), rnd(H, I, scale=0.02)
    gate, up, act = (torch.empty(BT, I, device="cuda", dtype=torch.bfloat16) for _ in range(3))
    dY = rnd(BT, H); d_act, d_gate, d_up = (torch.empty(BT, I, device="cuda", dtype=torch.bfloat16) for _ in range(3))
    ctx.call("ta_ctx_set_gemm_tuning", 0, 0, a.pair)

    def sep_f():
        ctx.call("ta_gemm_bf16", BT, I, H, 1.0, ptr(x), H, 0, ptr(Wg), H, 0, None, None, ptr(gate), I, stream_ptr())
        ctx.call("ta_gemm_bf16", BT, I, H, 1.0, ptr(x), H, 0, ptr(Wu), H, 0, None, None, ptr(up), I, stream_ptr())
        ctx.call("ta_silu_mul_fwd", ptr(gate), ptr(up), ptr(act), BT * I, stream_ptr())

    def fus_f():
        ctx.call("ta_swiglu_proj_fwd", ptr(x), ptr(Wg), ptr(Wu), None, None, None, ptr(gate), ptr(up), ptr(act), BT, H, I, 0, 1.0,
                 stream_ptr())

    def sep_b():
        ctx.call("ta_gemm_bf16", BT, I, H, 1.0, ptr(dY), H, 0, ptr(Wd), I, 1, None, None, ptr(d_act), I, stream_ptr())
        ctx.call("ta_silu_mul_bwd", ptr(d_act), ptr(gate), ptr(up), ptr(d_gate), ptr(d_up), BT * I, stream_ptr())

    def fus_b():
        ctx.call("ta_swiglu_down_bwd", ptr(dY), ptr(Wd), None, None, ptr(gate), ptr(up), ptr(d_gate), ptr(d_up), BT, H, I, 0, stream_ptr())

    fl = 2.0 * BT * I * H
    report("gate + up GEMMs + silu_mul_fwd", timeit(sep_f, a.iters, a.warmup, a.flush), flops=2 * fl, shape=[BT, H, I], pair=a.pair)
    report("fused gate/up SwiGLU forward", timeit(fus_f, a.iters, a.warmup, a.flush), flops=2 * fl, shape=[BT, H, I], pair=a.pair)
    report("down dX GEMM + silu_mul_bwd", timeit(sep_b, a.iters, a.warmup, a.flush), flops=fl, shape=[BT, H, I], pair=a.pair)
    report("fused down dX SwiGLU backward", timeit(fus_b, a.iters, a.warmup, a.flush), flops=fl, shape=[BT, H, I], pair=a.pair)
    ctx.call("ta_ctx_set_gemm_tuning", 0, 0, 0)


def kmeans(ctx, a):
    """Centroid merge (2048 vectors of dimension 512, k = 8 by default): reference-mode k-means and the seeded
    k-means++ / mass-ranked extension, whole call including its per-pass host synchronisation."""
    import ctypes
    N, D, k = a.N, a.D, a.k
    g = torch.Generator(device="cuda").manual_seed(0)
    centres = torch.randn(12, D, device="cuda", generator=g)
    vec = (centres[torch.randint(0, 12, (N,), device="cuda", generator=g)] + 0.1 * torch.randn(N, D, device="cuda", generator=g)).contiguous()
    mass = torch.rand(N, device="cuda", generator=g) + 0.1
    kk = min(k, N)
    cen, asg = torch.zeros(kk, D, device="cuda"), torch.zeros(N, dtype=torch.int32, device="cuda")
    kout, passes = ctypes.c_int(0), ctypes.c_int(0)
    f = lambda: ctx.call("ta_kmeans_merge", ptr(vec), N, D, k, 50, ptr(cen), ptr(asg), ctypes.byref(kout), ctypes.byref(passes), stream_ptr())
    t = timeit(f, a.iters, a.warmup, False)
    report("kmeans_merge (reference mode)", t, shape=[N, D, k], passes=passes.value)
    f2 = lambda: ctx.call("ta_kmeans_merge_ex", ptr(vec), ptr(mass), N, D, k, 50, 1, 7, 1, ptr(cen), ptr(asg), None, None,
                          ctypes.byref(kout), ctypes.byref(passes), stream_ptr())
    t = timeit(f2, a.iters, a.warmup, False)
    report("kmeans_merge_ex (k-means++ start, mass ranking)", t, shape=[N, D, k], passes=passes.value)


def rowops(ctx, a):
    rows, D, I = a.rows, a.D, a.I
    x, w, dy = rnd(rows, D), rnd(D), rnd(rows, D)
    out = torch.empty_like(x); rms = torch.empty(rows, device="cuda")
    g, u, d = rnd(rows, I), rnd(rows, I), rnd(rows, I)
    o1, o2 = torch.empty_like(g), torch.empty_like(g)
    n = rows * I
    t = timeit(lambda: ctx.call("ta_rms_norm_fwd", ptr(x), ptr(w), ptr(out), ptr(rms), rows, D, 1e-6, stream_ptr()), a.iters, a.warmup, a.flush)
    report("rms_norm_fwd", t, bytes_=rows * (4.0 * D + 4))
    t = timeit(lambda: ctx.call("ta_rms_norm_bwd", ptr(dy), ptr(x), ptr(w), ptr(rms), ptr(out), None, rows, D, stream_ptr()), a.iters, a.warmup, a.flush)
    report("rms_norm_bwd", t, bytes_=rows * (6.0 * D + 4))
    t = timeit(lambda: ctx.call("ta_silu_mul_fwd", ptr(g), ptr(u), ptr(o1), n, stream_ptr()), a.iters, a.warmup, a.flush)
    report("silu_mul_fwd", t, bytes_=6.0 * n)
    t = timeit(lambda: ctx.call("ta_silu_mul_bwd", ptr(d), ptr(g), ptr(u), ptr(o1), ptr(o2), n, stream_ptr()), a.iters, a.warmup, a.flush)
    report("silu_mul_bwd", t, bytes_=10.0 * n)
    acc = torch.zeros(D, device="cuda"); wt = torch.zeros(1, device="cuda")
    t = timeit(lambda: ctx.call("ta_centroid_accumulate", 0, ptr(x), ptr(dy), rows, D, ptr(acc), ptr(wt), stream_ptr()), a.iters, a.warmup, a.flush)
    report("centroid_accumulate", t, bytes_=4.0 * rows * D)
    H = 28
    q = rnd(rows, D)
    t = timeit(lambda: ctx.call("ta_rope", ptr(q), D // 128, None, 0, 1, rows, 128, 1e6, 0, stream_ptr()), a.iters, a.warmup, a.flush)
    report("rope", t, bytes_=4.0 * rows * D)


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="what", required=True)
    for name in ("attention", "gemm", "lora", "rowops", "skinny", "kmeans", "swiglu"):
        s = sub.add_parser(name)
        s.add_argument("--iters", type=int, default=10); s.add_argument("--warmup", type=int, default=3)
        s.add_argument("--flush", action="store_true")
        if name == "attention":
            for k, v in (("B", 1), ("T", 4096), ("Hq", 28), ("Hkv", 4), ("hd", 128)):
                s.add_argument("--" + k, type=int, default=v)
        elif name == "gemm":
            for k, v in (("M", 16384), ("N", 3584), ("K", 3584)):
                s.add_argument("--" + k, type=int, default=v)
            s.add_argument("--b-layout", type=int, default=0)
            s.add_argument("--tile", default="", help='force a tile "BN,MH" (experiment knob)')
            s.add_argument("--pair", type=int, default=0, help="256-wide tiles: 0 = library's choice, -1 = single-CTA kernel, 1 = 512x256 pair tiles, 2 = 256x256 pairs, 3 = 256x256 pairs with 128-wide k blocks")
            s.add_argument("--raster", default="", help='tile order "GROUP_M,GROUP_N" (experiment knob; 0 = default)')
        elif name == "kmeans":
            for k, v in (("N", 2048), ("D", 512), ("k", 8)):
                s.add_argument("--" + k, type=int, default=v)
        elif name in ("lora", "skinny"):
            for k, v in (("BT", 4096), ("in", 896), ("out", 896), ("rank", 16)):
                s.add_argument("--" + k, type=int, default=v)
        else:
            for k, v in (("rows", 16384), ("D", 3584), ("I", 18944)):
                s.add_argument("--" + k, type=int, default=v)
            if name == "swiglu":
                s.add_argument("--pair", type=int, default=0)
    a = ap.parse_args()
    ctx = ta.Context(0)
    {"attention": attention, "gemm": gemm, "lora": lora, "rowops": rowops, "skinny": skinny, "kmeans": kmeans, "swiglu": swiglu}[a.what](ctx, a)
    torch.cuda.synchronize()
    ctx.check_device()


if __name__ == "__main__":
    main()
