"""Generates the committed golden fixtures from the UNMODIFIED reference.

Run on a machine with a B200 and the compiled reference (oracle/_ref, built by `make -C oracle`):

    python tests/golden/make_golden.py <out_dir>

  ref_step_tiny.npz   seeded tiny Qwen2 (2 layers, hidden 256, 4/2 heads of 64, SwiGLU 512, vocab 512),
                      LoRA r=16 on q/k/v/o, batch 2 x 128, two AdamW steps: inputs (BF16 bit patterns,
                      FP32 LoRA masters, ids) and the reference's outputs (per-token loss, every gA/gB
                      before clipping, grad norm, masters after each step, both centroid snapshots)
  ref_ckpt_tiny/      the reference's own AdapterWriter output for the final masters of that run
                      (adapter.safetensors, adapter.json, train_state.json)
  ref_op_cfg2.npz     single LoRA-linear op (4096 x 896 -> 896, r16, alpha 32):
                      seed + reference outputs gA, gB in full and every 32nd row of y, dX (BF16 bits)
  ref_load_tiny.json  BaseLoader::load on the seeded model directory of tests/refcase.py hf_case(): the
                      derived config, base_sha and the SHA-256 of every loaded tensor's BF16 bytes
  kmeans_cfg1.npz     32 x 64 snapshot k-means through the reference CLI oracle/_ref/centroid-merge:
                      vector order as the reference enumerated it + merged centres (runs without a GPU)
"""
import os
import shutil
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path[:0] = [ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")]
import refcase as rc      # noqa: E402
import ta_oracle as o     # noqa: E402

TINY = dict(vocab=512, hidden=256, layers=2, hq=4, hkv=2, hd=64, inter=512)


def tiny_case():
    cfg = rc.tiny_cfg(**TINY)
    B, T, rank = 2, 128, 16
    base, adapter, toks, tgts = rc.make_case(cfg, B, T, rank, seed=11, steps=2, std=0.02, b_std=0.02)
    return cfg, B, T, rank, 32.0, 2e-4, base, adapter, toks, tgts


def make_step(out):
    cfg, B, T, rank, alpha, lr, base, adapter, toks, tgts = tiny_case()
    targets = ("q", "k", "v", "o")
    d = tempfile.mkdtemp()
    rc.write_case_dir(d + "/case", cfg, base, adapter, toks, tgts, B, T, rank, alpha, lr=lr, wd=0.01, grad_clip=1.0,
                      write_checkpoint=1)
    rc.run_harness("step", d + "/case", d + "/out")
    z = {"tokens": np.stack(toks), "targets": np.stack(tgts), "embed": o.bf16_bits(base["embed"]),
         "final_norm": o.bf16_bits(base["final_norm"]), "loss": rc.f32(d + "/out/loss.bin"),
         "grad_norm": rc.f32(d + "/out/grad_norm.bin")}
    for l, lw in enumerate(base["layers"]):
        for k in rc.LAYER_KEYS:
            z[f"l{l}_{k}"] = o.bf16_bits(lw[k])
        for t in targets:
            i, od = o.target_dims(cfg, t)
            z[f"l{l}_{t}_A"] = adapter[l][t].A_f32; z[f"l{l}_{t}_B"] = adapter[l][t].B_f32
            z[f"l{l}_{t}_gA"] = rc.f32(f"{d}/out/l{l}_lora_{t}_gA.bin", (rank, i))
            z[f"l{l}_{t}_gB"] = rc.f32(f"{d}/out/l{l}_lora_{t}_gB.bin", (od, rank))
            for s in range(2):
                z[f"s{s}_l{l}_{t}_A"] = rc.f32(f"{d}/out/after_step_{s}/l{l}_lora_{t}_A.bin", (rank, i))
                z[f"s{s}_l{l}_{t}_B"] = rc.f32(f"{d}/out/after_step_{s}/l{l}_lora_{t}_B.bin", (od, rank))
    for s in range(2):
        for nm, sub in (("intended", "centroids_intended"), ("asbuilt", "centroids_asbuilt")):
            c, w = o.read_snapshot_file(f"{d}/out/{sub}/step-{s + 1}.centroid")
            z[f"centroid_{nm}_{s}"] = c; z[f"centroid_{nm}_w_{s}"] = np.float32(w)
    np.savez_compressed(os.path.join(out, "ref_step_tiny.npz"), **z)
    ck = os.path.join(out, "ref_ckpt_tiny")
    shutil.rmtree(ck, ignore_errors=True)
    shutil.copytree(d + "/out/ckpt/step-final", ck)
    shutil.rmtree(d)


def make_op(out):
    seed, BT, ind, od, r = 2, 4096, 896, 896, 16
    rng = np.random.default_rng(seed)
    x = o.bf16_round(rng.standard_normal((BT, ind), dtype=np.float32))
    W = o.bf16_round(0.02 * rng.standard_normal((od, ind), dtype=np.float32))
    bound = np.sqrt(1.0 / ind)
    A = rng.uniform(-bound, bound, (r, ind)).astype(np.float32)
    Bm = (0.02 * rng.standard_normal((od, r))).astype(np.float32)
    dY = o.bf16_round(rng.standard_normal((BT, od), dtype=np.float32))
    d = tempfile.mkdtemp()
    os.makedirs(d + "/case")
    with open(d + "/case/cfg.txt", "w") as f:
        f.write(f"BT {BT}\nin {ind}\nout {od}\nrank {r}\nalpha 32\niters 20\n")
    for nm, a in (("x", x), ("W", W), ("dY", dY)):
        o.bf16_bits(a).astype("<u2").tofile(f"{d}/case/{nm}.bin")
    A.astype("<f4").tofile(d + "/case/A.bin"); Bm.astype("<f4").tofile(d + "/case/B.bin")
    log = rc.run_harness("op", d + "/case", d + "/out")
    np.savez_compressed(os.path.join(out, "ref_op_cfg2.npz"), seed=seed, shape=np.array([BT, ind, od, r]),
                        y=np.fromfile(d + "/out/y.bin", dtype="<u2").reshape(BT, od)[::32].copy(),
                        dX=np.fromfile(d + "/out/dX.bin", dtype="<u2").reshape(BT, ind)[::32].copy(), row_stride=np.int32(32),
                        gA=rc.f32(d + "/out/gA.bin", (r, ind)), gB=rc.f32(d + "/out/gB.bin", (od, r)))
    print(log.strip().splitlines()[0])
    shutil.rmtree(d)


def make_kmeans(out):
    vec, mass = o.cfg1_vectors(0)
    d = tempfile.mkdtemp()
    for i, (v, m) in enumerate(zip(vec, mass)):
        o.write_snapshot_file(f"{d}/step-{i:05d}.centroid", v, float(m))
    order = np.array([int(e.name[5:10]) for e in os.scandir(d) if e.name.endswith(".centroid")], dtype=np.int32)
    subprocess.run([os.path.join(ROOT, "oracle", "_ref", "centroid-merge"), d, "--out", d + "/merged.bin", "--clusters", "8"],
                   check=True, capture_output=True)
    np.savez_compressed(os.path.join(out, "kmeans_cfg1.npz"), seed=0, order=order, centers=o.read_merged_file(d + "/merged.bin"))
    shutil.rmtree(d)


def make_load(out):
    import hashlib
    import json
    d = tempfile.mkdtemp()
    cfg, _ = rc.hf_case(os.path.join(d, "hf"))
    rc.run_harness("load", os.path.join(d, "hf"), os.path.join(d, "ref"))
    conf = dict(l.split(None, 1) for l in open(os.path.join(d, "ref", "config.txt")).read().splitlines())
    hashes = {n[:-4]: hashlib.sha256(open(os.path.join(d, "ref", n), "rb").read()).hexdigest()
              for n in sorted(os.listdir(os.path.join(d, "ref"))) if n.endswith(".bin")}
    with open(os.path.join(out, "ref_load_tiny.json"), "w") as f:
        json.dump({"config": conf, "sha256_of_bf16_bytes": hashes}, f, indent=1, sort_keys=True)
    shutil.rmtree(d)


if __name__ == "__main__":
    out = sys.argv[1] if len(sys.argv) > 1 else HERE
    os.makedirs(out, exist_ok=True)
    which = sys.argv[2:] or ["kmeans", "step", "op", "load"]
    if "kmeans" in which:
        make_kmeans(out)
    if "step" in which:
        make_step(out)
    if "op" in which:
        make_op(out)
    if "load" in which:
        make_load(out)
    print("golden fixtures written to", out)
