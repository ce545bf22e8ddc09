"""CUDA path (through the C ABI) against the committed golden fixtures, i.e. outputs of the unmodified
reference (tests/golden/, made by tests/golden/make_golden.py).  Needs no reference binary at run time.

Bars: files and k-means bit-exact; the single LoRA-linear op (4096 x 896 -> 896, r16) at the stated tolerances
(gradients cosine >= 0.999 and max-rel <= 2e-2, BF16 outputs max-rel <= 2e-2); the 2-layer training step at
the measured BF16 noise floor documented in tests/test_gpu_trainer.py."""
import os

import numpy as np
import pytest
import torch

import refcase as rc
import ta_oracle as o
from tensor_adapt_b200 import ptr, stream_ptr
from test_oracle_golden import GOLD, TARGETS, load_tiny

pytestmark = pytest.mark.gpu


def dev_bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda().to(torch.bfloat16)


def test_cfg2_lora_linear_vs_reference_golden(ctx):
    z = np.load(os.path.join(GOLD, "ref_op_cfg2.npz"))
    BT, ind, od, r = (int(v) for v in z["shape"])
    rng = np.random.default_rng(int(z["seed"]))
    x = o.bf16_round(rng.standard_normal((BT, ind), dtype=np.float32))
    W = o.bf16_round(0.02 * rng.standard_normal((od, ind), dtype=np.float32))
    bound = np.sqrt(1.0 / ind)
    A = rng.uniform(-bound, bound, (r, ind)).astype(np.float32)
    Bm = (0.02 * rng.standard_normal((od, r))).astype(np.float32)
    dY = o.bf16_round(rng.standard_normal((BT, od), dtype=np.float32))
    xd, Wd, dYd, Ad, Bd = dev_bf16(x), dev_bf16(W), dev_bf16(dY), dev_bf16(o.bf16_round(A)), dev_bf16(o.bf16_round(Bm))
    y = torch.empty((BT, od), device="cuda", dtype=torch.bfloat16)
    dX = torch.empty((BT, ind), device="cuda", dtype=torch.bfloat16)
    gA = torch.zeros((r, ind), device="cuda"); gB = torch.zeros((od, r), device="cuda")
    ctx.call("ta_lora_linear_fwd", ptr(xd), ptr(Wd), None, ptr(Ad), ptr(Bd), None, ptr(y), BT, ind, od, r, 2.0, stream_ptr())
    ctx.call("ta_lora_linear_bwd", ptr(xd), ptr(dYd), ptr(Wd), ptr(Ad), ptr(Bd), ptr(dX), 0, ptr(gA), ptr(gB), BT, ind, od,
             r, 2.0, stream_ptr())
    torch.cuda.synchronize(); ctx.check_device()
    st = int(z["row_stride"])
    assert rc.relmax(y.float().cpu().numpy()[::st], o.bf16_from_bits(z["y"])) <= 2e-2
    assert rc.relmax(dX.float().cpu().numpy()[::st], o.bf16_from_bits(z["dX"])) <= 2e-2
    for got, ref in ((gA, z["gA"]), (gB, z["gB"])):
        got = got.cpu().numpy()
        assert rc.cosine(got, ref) >= 0.999 and rc.relmax(got, ref) <= 2e-2, (rc.cosine(got, ref), rc.relmax(got, ref))


def test_tiny_step_vs_reference_golden(ctx):
    from tensor_adapt_b200.trainer import AdaptTrainer, AdapterConfig
    z, cfg, base, adapter = load_tiny()
    B, T, rank, alpha, lr = 2, 128, 16, 32.0, 2e-4
    ac = AdapterConfig.defaults(rank=rank, alpha=alpha, targets=15, lr=lr, weight_decay=0.01, centroid_modes=3)
    tr = AdaptTrainer(ctx, rc.model_config(cfg), ac, B, T)
    rc.load_into_trainer(tr, cfg, base, adapter)
    for s in range(2):
        tr.zero_grad()
        tr.forward_backward(z["tokens"][s], z["targets"][s], B)
        if s == 0:
            loss = tr.download("cache.loss").ravel()
            np.testing.assert_allclose(loss, z["loss"], rtol=5e-3, atol=5e-3)
            for l in range(cfg.layers):
                for t in TARGETS:
                    for nm in ("gA", "gB"):
                        got, ref = tr.download(f"l{l}.lora.{t}.{nm}"), z[f"l{l}_{t}_{nm}"]
                        assert rc.cosine(got, ref) >= 0.998 and rc.relmax(got, ref) <= 8e-2, (l, t, nm)
        m = tr.optimizer_step(lr)
        if s == 0:
            assert abs(m.loss - o.mean_loss(z["loss"])) <= 1e-3 * m.loss
            assert abs(m.grad_norm_raw - z["grad_norm"][0]) <= 2e-2 * m.grad_norm_raw
        for l in range(cfg.layers):
            for t in TARGETS:
                assert np.abs(tr.download(f"l{l}.lora.{t}.A") - z[f"s{s}_l{l}_{t}_A"]).max() <= 2.2 * lr * (s + 1)
                assert np.abs(tr.download(f"l{l}.lora.{t}.B") - z[f"s{s}_l{l}_{t}_B"]).max() <= 2.2 * lr * (s + 1)
        for mode, nm in ((0, "intended"), (1, "asbuilt")):
            cen, w = tr.write_snapshot(s + 1, mode)
            ref = z[f"centroid_{nm}_{s}"]
            assert np.linalg.norm(cen - ref) <= 1.5e-2 * np.linalg.norm(ref), (nm, s)
            assert abs(w - z[f"centroid_{nm}_w_{s}"]) <= 1e-2 * w
    ctx.check_device()
    tr.close()


def test_checkpoint_files_byte_identical_to_reference(ctx, tmp_path):
    from tensor_adapt_b200.trainer import AdaptTrainer, AdapterConfig
    z, cfg, base, adapter = load_tiny()
    ac = AdapterConfig.defaults(rank=16, alpha=32.0, targets=15)
    tr = AdaptTrainer(ctx, rc.model_config(cfg), ac, 1, 128, domain="synthetic/domain")
    for l in range(cfg.layers):
        for t in TARGETS:
            tr.upload(f"l{l}.lora.{t}.A", z[f"s1_l{l}_{t}_A"]); tr.upload(f"l{l}.lora.{t}.B", z[f"s1_l{l}_{t}_B"])
    tr.set_meta("qwen2", "synthetic")
    tr.step_count, tr.tokens_seen = 2, 512
    tr.save_checkpoint(str(tmp_path / "ck"))
    ref = os.path.join(GOLD, "ref_ckpt_tiny")
    for f in ("adapter.safetensors", "adapter.json", "train_state.json"):
        assert (tmp_path / "ck" / f).read_bytes() == open(os.path.join(ref, f), "rb").read(), f
    tr.close()


def test_centroid_merge_dir_vs_reference_golden(ctx, tmp_path):
    """The 32 x 64 snapshot merge case through the file-level entry point (CentroidMerge::run): the reference CLI's
    merged centres are reproduced bit for bit when the vectors are enumerated in the same order."""
    from tensor_adapt_b200.trainer import centroid_merge
    z = np.load(os.path.join(GOLD, "kmeans_cfg1.npz"))
    vec, mass = o.cfg1_vectors(int(z["seed"]))
    d = tmp_path / "snaps"; d.mkdir()
    # one file per vector; names chosen so that ANY directory order can be mapped back
    for i in range(len(vec)):
        o.write_snapshot_file(str(d / f"step-{i:05d}.centroid"), vec[i], float(mass[i]))
    order = [int(e.name[5:10]) for e in os.scandir(d) if e.name.endswith(".centroid")]
    n, passes = centroid_merge(ctx, str(d), str(tmp_path / "merged.centroid"), 8)
    got = o.read_merged_file(str(tmp_path / "merged.centroid"))
    ref, _, ref_passes = o.kmeans_merge(vec[order], 8, 50)
    assert n == len(vec) and passes == ref_passes
    assert got.tobytes() == ref.tobytes()
    if order == list(z["order"]):
        assert got.tobytes() == z["centers"].tobytes()


def test_empty_and_degenerate_merge_inputs(ctx, tmp_path):
    import tensor_adapt_b200 as ta
    from tensor_adapt_b200.trainer import centroid_merge
    d = tmp_path / "empty"; d.mkdir()
    with pytest.raises(ta.TAError):
        centroid_merge(ctx, str(d), str(tmp_path / "x"), 4)          # "No .centroid files", as the reference throws
    o.write_snapshot_file(str(d / "step-1.centroid"), np.arange(8, dtype=np.float32), 1.0)
    n, passes = centroid_merge(ctx, str(d), str(tmp_path / "one.centroid"), 16)   # k clamps to N = 1
    got = o.read_merged_file(str(tmp_path / "one.centroid"))
    assert n == 1 and got.shape == (1, 8) and np.array_equal(got[0], np.arange(8, dtype=np.float32))
