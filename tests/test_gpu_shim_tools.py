"""The drop-in boundary, end to end: the reference's UNMODIFIED command-line tools (tools/centroid-merge.cpp,
tools/tensor-adapt.cpp) linked against the shim library (shim/*.cpp: the reference's own headers implemented
over the C ABI) and the CUDA library, run beside the same tools built from the reference's own sources.

  * centroid-merge: merged centres byte-identical to the reference binary's on the 32 x 64 snapshot case.
  * tensor-adapt: a short training run on a tiny Hugging Face style model directory writes the same set of files;
    adapter.json / train_state.json are byte-identical, the logged loss agrees within 1e-2 relative, the trained
    adapter tensors agree with the reference's (BF16 files; Adam's early steps amplify rounding noise on
    near-zero gradients, so agreement is asserted by cosine), and snapshot / merged centroid files have the
    reference's layout."""
import json
import os
import re
import subprocess

import numpy as np
import pytest

import refcase as rc
import ta_oracle as o

REF_DIR = os.path.join(rc.ROOT, "oracle", "_ref")
SHIM_MERGE, REF_MERGE = os.path.join(REF_DIR, "shim", "centroid-merge"), os.path.join(REF_DIR, "centroid-merge")
SHIM_ADAPT, REF_ADAPT = os.path.join(REF_DIR, "shim", "tensor-adapt"), os.path.join(REF_DIR, "tensor-adapt")

pytestmark = pytest.mark.gpu


def _run(cmd, **kw):
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, **kw)
    assert r.returncode == 0, f"{cmd[0]} failed:\n{r.stderr[-3000:]}"
    return r.stderr + r.stdout


@pytest.mark.skipif(not (os.path.exists(SHIM_MERGE) and os.path.exists(REF_MERGE)), reason="shim / reference tools not built")
def test_reference_centroid_merge_tool_on_the_shim_is_byte_identical(tmp_path):
    vec, mass = o.cfg1_vectors(0)
    d = tmp_path / "snaps"; d.mkdir()
    for i in range(len(vec)):
        o.write_snapshot_file(str(d / f"step-{i:05d}.centroid"), vec[i], float(mass[i]))
    _run([REF_MERGE, str(d), "--out", str(tmp_path / "ref.centroid"), "--clusters", "8"])
    log = _run([SHIM_MERGE, str(d), "--out", str(tmp_path / "shim.centroid"), "--clusters", "8"])
    assert (tmp_path / "shim.centroid").read_bytes() == (tmp_path / "ref.centroid").read_bytes()
    assert "merged 2048 snapshots" in log
    # error behaviour of the tool is the reference's: exit code 1 and "error: No .centroid files in <dir>"
    e = tmp_path / "empty"; e.mkdir()
    r = subprocess.run([SHIM_MERGE, str(e), "--out", str(tmp_path / "x")], capture_output=True, text=True)
    assert r.returncode == 1 and "No .centroid files" in r.stderr


def _tensors(path):
    """{name: float32 array} of a BF16 / F32 safetensors file."""
    b = open(path, "rb").read()
    n = int.from_bytes(b[:8], "little")
    hdr = json.loads(b[8:8 + n])
    out = {}
    for k, v in hdr.items():
        if k == "__metadata__":
            continue
        raw = b[8 + n + v["data_offsets"][0]:8 + n + v["data_offsets"][1]]
        a = o.bf16_from_bits(np.frombuffer(raw, dtype="<u2")) if v["dtype"] == "BF16" else np.frombuffer(raw, dtype="<f4")
        out[k] = a.reshape(v["shape"])
    return out


@pytest.mark.skipif(not (os.path.exists(SHIM_ADAPT) and os.path.exists(REF_ADAPT)), reason="shim / reference tools not built")
def test_reference_tensor_adapt_tool_on_the_shim_trains_like_the_reference(tmp_path):
    cfg, _ = rc.hf_case(str(tmp_path / "model"), shards=2)
    rng = np.random.default_rng(3)
    toks = rng.integers(0, cfg.vocab, size=4096).astype("<u4")
    # a random stream has no assistant turns, so every target is masked to -1; as in the reference such tokens still
    # carry loss = logsumexp and gradient softmax / rows (src/backend/cuda/ops.cu:997-1010), so training proceeds
    toks.tofile(str(tmp_path / "train.bin"))
    steps, B, T = 20, 2, 64
    outs = {}
    for name, exe in (("ref", REF_ADAPT), ("shim", SHIM_ADAPT)):
        out = tmp_path / f"out_{name}"
        log = _run([exe, "--base", str(tmp_path / "model"), "--data", str(tmp_path / "train.bin"), "--domain", "synthetic/domain",
                    "--output", str(out), "--tokens", str(steps * B * T), "--ckpt-every", "10", "--rank", "16", "--alpha", "32",
                    "--lr", "1e-3", "--warmup", "2", "--batch", str(B), "--seq", str(T)])
        outs[name] = (out, log)
    (ro, rlog), (so, slog) = outs["ref"], outs["shim"]
    # same files in the same places
    listing = lambda d: sorted(os.path.relpath(os.path.join(p, f), d) for p, _, fs in os.walk(d) for f in fs)
    assert [f for f in listing(so) if not f.endswith("optimizer.safetensors")] == listing(ro)
    for f in ("adapter.json", "step-10/adapter.json", "step-10/train_state.json", "step-20/train_state.json"):
        assert (so / f).read_bytes() == (ro / f).read_bytes(), f
    # the step lines the tool logs every 10 steps
    pat = re.compile(r"\[step (\d+)/(\d+)\] loss=([0-9.eE+-]+) lr=([0-9.eE+-]+) grad=([0-9.eE+-]+) tok=(\d+)")
    rl, sl = pat.findall(rlog), pat.findall(slog)
    assert len(rl) == len(sl) == 2
    for a, b in zip(rl, sl):
        assert a[0] == b[0] and a[1] == b[1] and a[5] == b[5]
        assert abs(float(a[2]) - float(b[2])) <= 1e-2 * float(a[2])          # loss
        assert abs(float(a[3]) - float(b[3])) <= 1e-6 * float(a[3]) + 1e-12  # cosine schedule
    # all-masked batches (no assistant turns in a random stream) still carry the reference's gradient; adapters move alike
    tr, ts = _tensors(ro / "adapter.safetensors"), _tensors(so / "adapter.safetensors")
    assert sorted(tr) == sorted(ts)
    for k in tr:
        assert tr[k].shape == ts[k].shape
        assert rc.cosine(ts[k], tr[k]) >= 0.98, (k, rc.cosine(ts[k], tr[k]))
    # centroid files: same layout and dimension (the shipped reference computes its as-built sum; the shim the documented one)
    for f in ("centroids/step-10.centroid", "centroids/step-20.centroid"):
        cs, ws = o.read_snapshot_file(str(so / f)); cr, wr = o.read_snapshot_file(str(ro / f))
        assert cs.shape == cr.shape and np.isfinite(cs).all() and ws > 0
    ms, mr = o.read_merged_file(str(so / "adapter.centroid")), o.read_merged_file(str(ro / "adapter.centroid"))
    assert ms.shape == mr.shape


@pytest.mark.skipif(not (os.path.exists(SHIM_ADAPT) and os.path.exists(REF_ADAPT)), reason="shim / reference tools not built")
def test_shim_built_tool_reproduces_the_shipped_centroid_when_asked(tmp_path):
    """TA_SHIM_CENTROID=asbuilt makes the shim accumulate what the shipped reference trainer computes
    (FP32 copies re-read as BF16, src/trainer/adapt_trainer.cu:210-232): snapshot files then agree."""
    cfg, _ = rc.hf_case(str(tmp_path / "model"), shards=1)
    np.random.default_rng(4).integers(0, cfg.vocab, size=2048).astype("<u4").tofile(str(tmp_path / "train.bin"))
    res = {}
    for name, exe in (("ref", REF_ADAPT), ("shim", SHIM_ADAPT)):
        out = tmp_path / f"out_{name}"
        _run([exe, "--base", str(tmp_path / "model"), "--data", str(tmp_path / "train.bin"), "--domain", "d", "--output", str(out),
              "--tokens", "256", "--ckpt-every", "1", "--rank", "16", "--alpha", "32", "--lr", "2e-4", "--warmup", "1", "--batch", "2",
              "--seq", "64"], env=dict(os.environ, TA_SHIM_CENTROID="asbuilt"))
        res[name] = o.read_snapshot_file(str(out / "centroids" / "step-1.centroid"))
    (cs, ws), (cr, wr) = res["shim"], res["ref"]
    assert abs(ws - wr) <= 2e-2 * wr
    assert np.linalg.norm(cs - cr) <= 3e-2 * np.linalg.norm(cr)
    assert not cs[0::2].any() and not cr[0::2].any()      # the as-built sum only ever fills odd positions
