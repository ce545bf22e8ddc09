"""Multi-vector snapshot banks (an extension the reference's README describes, README.md:73-79, and has no code
for): a snapshot file holds several vectors as the reference's single-vector record repeated back to back.

CPU part: the file format round-trips, and the UNMODIFIED reference binary (oracle/_ref/centroid-merge) still reads
such files - it sees the first record of each, so the format is backward compatible.
GPU part: the extended merge clusters every record of every file, bit-exactly as the oracle restatement does on
the vectors enumerated in the same order; the reference-mode merge keeps the reference's first-record behaviour;
the trainer's per-layer bank agrees with the oracle's per-layer accumulation and adds up to the global accumulator."""
import os
import subprocess

import numpy as np
import pytest

import refcase as rc
import ta_oracle as o

REF_MERGE = os.path.join(rc.ROOT, "oracle", "_ref", "centroid-merge")


def _bank_dir(d, n_files=32, per_file=64, seed=0):
    vec, mass = o.cfg1_vectors(seed, n_snap=n_files, per_snap=per_file)
    os.makedirs(d)
    for i in range(n_files):
        o.write_bank_file(os.path.join(d, f"step-{i:05d}.centroid"), vec[i * per_file:(i + 1) * per_file], mass[i * per_file:(i + 1) * per_file])
    order = [int(e.name[5:10]) for e in os.scandir(d) if e.name.endswith(".centroid")]
    return vec.reshape(n_files, per_file, -1), mass.reshape(n_files, per_file), order


def test_bank_file_round_trip_and_single_record_equals_reference_snapshot(tmp_path):
    v = np.random.default_rng(0).standard_normal((5, 16)).astype(np.float32)
    w = np.arange(1, 6, dtype=np.float32)
    p = str(tmp_path / "b.centroid")
    o.write_bank_file(p, v, w)
    v2, w2 = o.read_bank_file(p)
    assert np.array_equal(v, v2) and np.array_equal(w, w2)
    c, w0 = o.read_snapshot_file(p)                          # the single-vector reader sees record 0
    assert np.array_equal(c, v[0]) and w0 == 1.0
    o.write_bank_file(p, v[:1], w[:1]); q = str(tmp_path / "s.centroid")
    o.write_snapshot_file(q, v[0], 1.0)
    assert open(p, "rb").read() == open(q, "rb").read()


@pytest.mark.skipif(not os.path.exists(REF_MERGE), reason="reference centroid-merge binary not built")
def test_reference_binary_reads_the_first_record_of_a_bank(tmp_path):
    vec, _, order = _bank_dir(str(tmp_path / "banks"), n_files=16, per_file=8)
    r = subprocess.run([REF_MERGE, str(tmp_path / "banks"), "--out", str(tmp_path / "m.bin"), "--clusters", "4"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    want, _, _ = o.kmeans_merge(vec[order, 0, :], 4, 50)
    assert o.read_merged_file(str(tmp_path / "m.bin")).tobytes() == want.tobytes()


@pytest.mark.gpu
def test_extended_merge_clusters_every_record_bit_exactly(ctx, tmp_path):
    from tensor_adapt_b200.trainer import centroid_merge, centroid_merge_ranked
    vec, mass, order = _bank_dir(str(tmp_path / "banks"))                      # 32 files x 64 vectors of dimension 512
    flat_v = vec[order].reshape(-1, vec.shape[-1]); flat_m = mass[order].reshape(-1)
    n, passes = centroid_merge_ranked(ctx, str(tmp_path / "banks"), str(tmp_path / "bank.bin"), k=8, seed=7)
    want_c, _, want_it, _, _ = o.kmeans_merge_ex(flat_v, flat_m, 8, 7)
    assert n == 2048 and passes == want_it
    assert o.read_merged_file(str(tmp_path / "bank.bin")).tobytes() == want_c.tobytes()
    # the reference-mode merge keeps the reference's reading: first record of each file
    n1, _ = centroid_merge(ctx, str(tmp_path / "banks"), str(tmp_path / "ref.bin"), 8)
    want1, _, _ = o.kmeans_merge(vec[order, 0, :], 8, 50)
    assert n1 == 32 and o.read_merged_file(str(tmp_path / "ref.bin")).tobytes() == want1.tobytes()


@pytest.mark.gpu
def test_trainer_per_layer_bank_matches_oracle_and_sums_to_the_global_accumulator(ctx, tmp_path):
    from tensor_adapt_b200.trainer import AdaptTrainer, AdapterConfig
    cfg = rc.tiny_cfg(hidden=256, hq=4, hkv=2, hd=64, inter=512, layers=3)
    B, T, rank, alpha = 2, 128, 16, 32.0
    base, adapter, toks, tgts = rc.make_case(cfg, B, T, rank, seed=12, std=0.02, b_std=0.02)
    ac = AdapterConfig.defaults(rank=rank, alpha=alpha, lr=2e-4, centroid_modes=1 | 4)
    tr = AdaptTrainer(ctx, rc.model_config(cfg), ac, B, T)
    rc.load_into_trainer(tr, cfg, base, adapter)
    tr.zero_grad(); tr.forward_backward(toks[0], tgts[0], B)
    path = str(tmp_path / "step-1.centroid")
    cen, w = tr.write_snapshot_bank(path)
    raw_acc, raw_w = tr.download("centroid_bank.acc"), tr.download("centroid_bank.weight").ravel()
    glob_acc, glob_w = tr.download("centroid.acc").ravel(), float(tr.download("centroid.weight").ravel()[0])
    ctx.check_device(); tr.close()
    # the layers' sums add up to the single accumulator the reference keeps
    assert abs(raw_w.sum() - glob_w) <= 1e-5 * glob_w
    assert np.abs(raw_acc.sum(0) - glob_acc).max() <= 1e-4 * np.abs(glob_acc).max()
    # file = one reference-layout record per layer
    fv, fw = o.read_bank_file(path)
    assert fv.shape == (cfg.layers, cfg.hidden) and np.array_equal(fv, cen) and np.array_equal(fw, w)
    # against the oracle's step (BF16 noise of the backward between the two implementations, as for the global centroid)
    ref = o.train_step(cfg, base, adapter, toks[0], tgts[0], B, T, alpha=alpha, rank=rank, lr=2e-4, step=1)
    want_c, want_w = o.layer_bank([ref["fwd"]["layer_cache"][l]["x_normed"] for l in range(cfg.layers)],
                                  [ref["layer_grads"][l]["dx_attn_in"] for l in range(cfg.layers)])
    for l in range(cfg.layers):
        assert abs(w[l] - want_w[l]) <= 2e-2 * want_w[l]
        assert np.linalg.norm(cen[l] - want_c[l]) <= 3e-2 * np.linalg.norm(want_c[l]), l
    # a trainer created without the bank refuses the call
    tr2 = AdaptTrainer(ctx, rc.model_config(cfg), AdapterConfig.defaults(rank=rank, alpha=alpha), B, T)
    import tensor_adapt_b200 as ta
    with pytest.raises(ta.TAError):
        tr2.write_snapshot_bank()
    tr2.close()
