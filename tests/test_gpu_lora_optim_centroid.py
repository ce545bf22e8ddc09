"""LoRA linear fwd/bwd (the 4096 x 896 -> 896 rank-16 single-op case and small ragged cases), the flat-arena optimiser, the
device centroid accumulator and the device k-means, each through the C ABI against the oracle.

Tolerances (config 2's, from the north star): LoRA gradients cosine >= 0.999 and
max|err| <= 2e-2 * max|ref|; BF16 activations max|err| <= 2e-2 * max|ref|; centroid vector relative
L2 <= 1e-3; k-means assignments and centres bit-exact."""
import ctypes
import os

import numpy as np
import pytest
import torch

import ta_oracle as o
from tensor_adapt_b200 import ptr, stream_ptr

pytestmark = pytest.mark.gpu


def dev_bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda().to(torch.bfloat16)


def dev_f32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def relmax(out, ref):
    return float(np.abs(out - ref).max() / (np.abs(ref).max() + 1e-30))


def cosine(a, b):
    a = a.ravel().astype(np.float64); b = b.ravel().astype(np.float64)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300))


def lora_case(BT, ind, outd, r, seed=0):
    rng = np.random.default_rng(seed)
    x = o.bf16_round(rng.standard_normal((BT, ind), dtype=np.float32))
    W = o.bf16_round(0.02 * rng.standard_normal((outd, ind), dtype=np.float32))
    bound = np.sqrt(1.0 / ind)
    A = rng.uniform(-bound, bound, (r, ind)).astype(np.float32)
    B = (0.02 * rng.standard_normal((outd, r))).astype(np.float32)
    dY = o.bf16_round(rng.standard_normal((BT, outd), dtype=np.float32))
    bias = o.bf16_round(0.02 * rng.standard_normal(outd, dtype=np.float32))
    return x, W, A, B, dY, bias


@pytest.mark.parametrize("BT,ind,outd,r,scale", [(4096, 896, 896, 16, 2.0), (200, 128, 256, 64, 2.0),
                                                  (1000, 896, 128, 16, 0.75), (384, 4864, 896, 32, 1.0)])
def test_lora_linear_fwd_bwd(ctx, BT, ind, outd, r, scale):
    x, W, A, B, dY, bias = lora_case(BT, ind, outd, r)
    lp = o.LoraPair(A, B)
    y_ref = o.apply_lora_fwd(lp, x, o.add_bias(o.proj_fwd(W, x), bias), scale)
    dX0 = o.bf16_round(np.random.default_rng(9).standard_normal((BT, ind), dtype=np.float32))
    dx_ref = o.apply_lora_bwd(lp, x, dY, o.proj_bwd_x(W, dY, dX0), scale)

    xd, Wd, dYd, bd = dev_bf16(x), dev_bf16(W), dev_bf16(dY), dev_bf16(bias)
    Ad, Bd = dev_bf16(lp.A_bf16), dev_bf16(lp.B_bf16)
    y = torch.full((BT, outd), float("nan"), device="cuda", dtype=torch.bfloat16)
    ctx.call("ta_lora_linear_fwd", ptr(xd), ptr(Wd), ptr(bd), ptr(Ad), ptr(Bd), None, ptr(y), BT, ind, outd, r, scale,
             stream_ptr())
    dX = dev_bf16(dX0)
    gA = torch.zeros((r, ind), device="cuda"); gB = torch.zeros((outd, r), device="cuda")
    ctx.call("ta_lora_linear_bwd", ptr(xd), ptr(dYd), ptr(Wd), ptr(Ad), ptr(Bd), ptr(dX), 1, ptr(gA), ptr(gB), BT, ind,
             outd, r, scale, stream_ptr())
    torch.cuda.synchronize(); ctx.check_device()
    assert relmax(y.float().cpu().numpy(), y_ref) <= 2e-2
    assert relmax(dX.float().cpu().numpy(), dx_ref) <= 2e-2
    for name, got, ref in (("gA", gA, lp.gA), ("gB", gB, lp.gB)):
        got = got.cpu().numpy()
        assert cosine(got, ref) >= 0.999 and relmax(got, ref) <= 2e-2, (name, cosine(got, ref), relmax(got, ref))
    # gradients accumulate (+=) and are reproducible bit for bit
    gA2 = torch.zeros_like(gA); gB2 = torch.zeros_like(gB); dX2 = dev_bf16(dX0)
    for _ in range(2):
        ctx.call("ta_lora_linear_bwd", ptr(xd), ptr(dYd), ptr(Wd), ptr(Ad), ptr(Bd), ptr(dX2), 0, ptr(gA2), ptr(gB2), BT,
                 ind, outd, r, scale, stream_ptr())
    torch.cuda.synchronize()
    assert torch.allclose(gA2, 2 * gA, rtol=1e-6, atol=1e-7) and torch.allclose(gB2, 2 * gB, rtol=1e-6, atol=1e-7)


def test_lora_linear_without_adapter(ctx):
    x, W, _, _, dY, _ = lora_case(300, 256, 384, 16)
    xd, Wd, dYd = dev_bf16(x), dev_bf16(W), dev_bf16(dY)
    y = torch.empty((300, 384), device="cuda", dtype=torch.bfloat16)
    ctx.call("ta_lora_linear_fwd", ptr(xd), ptr(Wd), None, None, None, None, ptr(y), 300, 256, 384, 0, 1.0, stream_ptr())
    dX = torch.empty((300, 256), device="cuda", dtype=torch.bfloat16)
    ctx.call("ta_lora_linear_bwd", None, ptr(dYd), ptr(Wd), None, None, ptr(dX), 0, None, None, 300, 256, 384, 0, 1.0,
             stream_ptr())
    torch.cuda.synchronize()
    assert relmax(y.float().cpu().numpy(), o.proj_fwd(W, x)) <= 1e-2
    assert relmax(dX.float().cpu().numpy(), o.proj_bwd_x(W, dY)) <= 1e-2


def test_gradnorm_clip_adamw(ctx):
    rng = np.random.default_rng(5)
    n = 100_003
    master = rng.standard_normal(n).astype(np.float32) * 0.05
    grad = rng.standard_normal(n).astype(np.float32) * 0.01
    m = np.zeros(n, np.float32); v = np.zeros(n, np.float32)
    md, gd, mmd, vd = dev_f32(master), dev_f32(grad), dev_f32(m), dev_f32(v)
    wd_ = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    stats = torch.zeros(2, device="cuda")
    ref_master = master.copy(); ref_m = m.copy(); ref_v = v.copy(); ref_g = grad.copy()
    for step in (1, 2, 3):
        norm = float(np.sqrt(np.sum(ref_g.astype(np.float64) ** 2)))
        g_used = ref_g * np.float32(1.0 / (norm + 1e-6)) if norm > 1.0 else ref_g
        ref_w = o.adamw_step(ref_master, ref_m, ref_v, g_used, 2e-4, 0.9, 0.999, 1e-8, 0.01, step)
        ctx.call("ta_gradnorm_clip_adamw", ptr(md), ptr(wd_), ptr(mmd), ptr(vd), ptr(gd), n, 2e-4, 0.9, 0.999, 1e-8, 0.01,
                 step, 1.0, ptr(stats), 0, stream_ptr())
        torch.cuda.synchronize()
        assert abs(stats[0].item() - norm) <= 1e-5 * norm
        np.testing.assert_allclose(md.cpu().numpy(), ref_master, rtol=2e-6, atol=1e-9)
        np.testing.assert_allclose(mmd.cpu().numpy(), ref_m, rtol=2e-6, atol=1e-12)
        np.testing.assert_allclose(vd.cpu().numpy(), ref_v, rtol=2e-6, atol=1e-15)
        assert np.abs(wd_.float().cpu().numpy() - ref_w).max() <= 2 ** -8 * np.abs(ref_w).max()
    # the single-tensor form and the norm accumulator
    acc = torch.zeros(1, device="cuda")
    ctx.call("ta_sum_sq_into", ptr(gd), ptr(acc), n, stream_ptr())
    ctx.call("ta_sum_sq_into", ptr(gd), ptr(acc), n, stream_ptr())
    torch.cuda.synchronize()
    assert abs(acc.item() - 2 * np.sum(grad.astype(np.float64) ** 2)) <= 1e-5 * acc.item()


@pytest.mark.parametrize("BT,D", [(8192, 896), (333, 3584), (64, 64)])
@pytest.mark.parametrize("mode", [0, 1])
def test_centroid_accumulate(ctx, BT, D, mode):
    rng = np.random.default_rng(6)
    h = o.bf16_round(rng.standard_normal((BT, D), dtype=np.float32))
    g = o.bf16_round(1e-3 * rng.standard_normal((BT, D), dtype=np.float32))
    ref = o.CentroidAccumulator(D)
    acc = torch.zeros(D, device="cuda"); w = torch.zeros(1, device="cuda")
    hd_, gd_ = dev_bf16(h), dev_bf16(g)
    for _ in range(2):   # state accumulates across calls (all layers share it)
        ref.accumulate(h, g, "intended" if mode == 0 else "asbuilt")
        ctx.call("ta_centroid_accumulate", mode, ptr(hd_), ptr(gd_), BT, D, ptr(acc), ptr(w), stream_ptr())
    torch.cuda.synchronize()
    got = acc.cpu().numpy()
    # FP64 restatement as the arbiter: the device (tree sums) must be at least as close to it as 1e-3,
    # the criterion stated for centroid vectors (relative L2)
    assert abs(w.item() - ref.weight[0]) <= 1e-4 * ref.weight[0]
    rel = np.linalg.norm(got - ref.acc) / (np.linalg.norm(ref.acc) + 1e-30)
    assert rel <= 1e-3, rel
    if mode == 1:
        assert np.all(got[0::2] == 0)


@pytest.mark.parametrize("N,D,k,seed", [(2048, 512, 8, 0), (32, 896, 16, 1), (5, 64, 16, 2), (300, 40, 7, 3)])
def test_kmeans_merge_bit_exact(ctx, N, D, k, seed):
    if (N, D) == (2048, 512):
        vec, _ = o.cfg1_vectors(seed)           # the 32 x 64 snapshot merge case
    else:
        rng = np.random.default_rng(seed)
        vec = rng.standard_normal((N, D)).astype(np.float32)
        vec[N // 2:] = vec[: N - N // 2]        # duplicates: ties and (for k > distinct) empty clusters
    ref_c, ref_a, ref_it = o.kmeans_merge(vec, k, 50)
    vd = dev_f32(vec)
    kk = min(k, N)
    centers = torch.empty((kk, D), device="cuda"); assign = torch.empty(N, device="cuda", dtype=torch.int32)
    kout = ctypes.c_int(0); passes = ctypes.c_int(0)
    ctx.call("ta_kmeans_merge", ptr(vd), N, D, k, 50, ptr(centers), ptr(assign), ctypes.byref(kout), ctypes.byref(passes),
             stream_ptr())
    torch.cuda.synchronize()
    assert kout.value == kk and passes.value == ref_it
    assert np.array_equal(assign.cpu().numpy(), ref_a)
    assert centers.cpu().numpy().tobytes() == ref_c.tobytes()


@pytest.mark.parametrize("N,D,k,seed", [(2048, 512, 8, 0), (100, 64, 16, 7), (5, 32, 8, 3), (513, 96, 3, 11)])
def test_kmeans_plusplus_and_mass_ranking_bit_exact(ctx, N, D, k, seed):
    """Extension (no reference code): seeded k-means++ start + Lloyd + ranking by gradient mass equals the
    oracle's restatement bit for bit - chosen start vectors, centres, labels, FP64 cluster masses."""
    if (N, D) == (2048, 512):
        vec, mass = o.cfg1_vectors(seed)
    else:
        rng = np.random.default_rng(seed)
        vec = rng.standard_normal((N, D)).astype(np.float32)
        mass = rng.lognormal(0, 1, N).astype(np.float32)
        vec[N // 2] = vec[0]                                            # duplicates: zero distances in the CDF
    want_c, want_a, want_it, want_tot, want_idx = o.kmeans_merge_ex(vec, mass, k, seed)
    kk = min(k, N)
    vd, md = torch.from_numpy(vec).cuda(), torch.from_numpy(mass).cuda()
    centers = torch.zeros(kk, D, device="cuda"); assign = torch.zeros(N, dtype=torch.int32, device="cuda")
    tot = torch.zeros(kk, dtype=torch.float64, device="cuda"); idx = torch.zeros(kk, dtype=torch.int32, device="cuda")
    kout, passes = ctypes.c_int(0), ctypes.c_int(0)
    ctx.call("ta_kmeans_merge_ex", ptr(vd), ptr(md), N, D, k, 50, 1, seed, 1, ptr(centers), ptr(assign), ptr(tot), ptr(idx),
             ctypes.byref(kout), ctypes.byref(passes), stream_ptr())
    torch.cuda.synchronize()
    assert kout.value == kk and passes.value == want_it
    np.testing.assert_array_equal(idx.cpu().numpy(), want_idx)
    np.testing.assert_array_equal(assign.cpu().numpy(), want_a)
    np.testing.assert_array_equal(centers.cpu().numpy(), want_c)
    np.testing.assert_array_equal(tot.cpu().numpy(), want_tot)
    assert np.all(np.diff(tot.cpu().numpy()) <= 0)                      # ranked: heaviest cluster first
    # even-spread start + no ranking through the same entry point == the reference-mode merge
    ref_c, ref_a, ref_it = o.kmeans_merge(vec, k, 50)
    ctx.call("ta_kmeans_merge_ex", ptr(vd), None, N, D, k, 50, 0, 0, 0, ptr(centers), ptr(assign), None, None,
             ctypes.byref(kout), ctypes.byref(passes), stream_ptr())
    torch.cuda.synchronize()
    np.testing.assert_array_equal(centers.cpu().numpy(), ref_c)
    np.testing.assert_array_equal(assign.cpu().numpy(), ref_a)


def test_ranked_merge_of_a_snapshot_directory(ctx, tmp_path):
    from tensor_adapt_b200.trainer import centroid_merge_ranked
    vec, mass = o.cfg1_vectors(2, n_snap=8, per_snap=32)
    d = tmp_path / "centroids"; d.mkdir()
    for i, (v, m) in enumerate(zip(vec, mass)):
        o.write_snapshot_file(str(d / f"step-{i:05d}.centroid"), v, float(m))
    order = np.array([int(e.name[5:10]) for e in os.scandir(d) if e.name.endswith(".centroid")])
    n, passes = centroid_merge_ranked(ctx, str(d), str(tmp_path / "bank.bin"), k=8, seed=5)
    want_c, _, want_it, _, _ = o.kmeans_merge_ex(vec[order], mass[order], 8, 5)
    assert n == len(vec) and passes == want_it
    np.testing.assert_array_equal(o.read_merged_file(str(tmp_path / "bank.bin")), want_c)
