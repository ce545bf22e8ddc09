"""Real-weight loading and resume on the GPU: a Hugging Face style directory (BF16 and F32 tensors,
one file or shards) lands bit-exactly in the weight arena; a checkpoint + optimizer.safetensors
continues bit-exactly; a reference-format checkpoint (BF16 only) restores masters and counters."""
import os

import numpy as np
import pytest

import refcase as rc
import ta_oracle as o

pytestmark = pytest.mark.gpu


def _case(tie=True):
    cfg = rc.tiny_cfg(hidden=128, hq=2, hkv=1, hd=64, inter=256, vocab=320, layers=2)
    cfg.tie = tie
    base, adapter, toks, tgts = rc.make_case(cfg, 2, 64, 16, seed=11, steps=4, std=0.05, b_std=0.05)
    return cfg, base, adapter, toks, tgts


def _trainer(ctx, cfg, rank=16, alpha=32.0, targets=15):
    from tensor_adapt_b200.trainer import AdaptTrainer, AdapterConfig
    ac = AdapterConfig.defaults(rank=rank, alpha=alpha, targets=targets, lr=1e-3, weight_decay=0.01, centroid_modes=3)
    return AdaptTrainer(ctx, rc.model_config(cfg), ac, 2, 64)


@pytest.mark.parametrize("shards,tie", [(1, True), (3, False)])
def test_load_base_matches_uploaded_tensors(ctx, tmp_path, shards, tie):
    cfg, base, adapter, toks, tgts = _case(tie)
    d = str(tmp_path / "hf")
    f32_names = {"model.layers.1.self_attn.q_proj.weight", "model.norm.weight", "model.layers.0.mlp.down_proj.weight"}
    rng = np.random.default_rng(5)
    # F32 tensors with values that are NOT BF16-representable: the loader must round them (RNE)
    base["layers"][1]["q_w"] = (rng.standard_normal(base["layers"][1]["q_w"].shape) * 0.05).astype(np.float32)
    base["layers"][0]["down_w"] = (rng.standard_normal(base["layers"][0]["down_w"].shape) * 0.05).astype(np.float32)
    o.write_hf_dir(d, cfg, base, shards=shards, f32_names=f32_names)
    tr = _trainer(ctx, cfg)
    tr.load_base(d)
    for name, want in (("embed", base["embed"]), ("final_norm", base["final_norm"])) + ((("lm_head", base["lm_head"]),) if not tie else ()):
        np.testing.assert_array_equal(tr.download(name).reshape(want.shape), o.bf16_round(want))
    for l, lw in enumerate(base["layers"]):
        for k in rc.LAYER_KEYS:
            np.testing.assert_array_equal(tr.download(f"l{l}.{k}").reshape(lw[k].shape), o.bf16_round(lw[k]), err_msg=f"l{l}.{k}")
    # the loaded base trains: same loss as a trainer fed through upload()
    tr2 = _trainer(ctx, cfg)
    for lw in base["layers"]:
        for k in ("q_w", "down_w"):
            lw[k] = o.bf16_round(lw[k])
    rc.load_into_trainer(tr2, cfg, base, adapter)
    for l in range(cfg.layers):
        for t, lp in adapter[l].items():
            tr.upload(f"l{l}.lora.{t}.A", lp.A_f32); tr.upload(f"l{l}.lora.{t}.B", lp.B_f32)
    tr.sync_working()
    m1, m2 = tr.step(toks[0], tgts[0], 2, lr=1e-3), tr2.step(toks[0], tgts[0], 2, lr=1e-3)
    assert m1.loss == m2.loss and m1.grad_norm_raw == m2.grad_norm_raw
    # adapter.json records the model_type and the directory's sha
    out = str(tmp_path / "ck")
    tr.save_checkpoint(out)
    import json
    j = json.load(open(os.path.join(out, "adapter.json")))
    assert j["architecture"] == "qwen2" and j["base_sha"] == o.base_sha(d)
    tr.close(); tr2.close()


def test_load_base_rejects_mismatch_and_f16(ctx, tmp_path):
    from tensor_adapt_b200 import TAError
    cfg, base, *_ = _case()
    d = str(tmp_path / "hf")
    o.write_hf_dir(d, cfg, base)
    cfg2 = rc.tiny_cfg(hidden=128, hq=2, hkv=1, hd=64, inter=256, vocab=320, layers=3)
    tr = _trainer(ctx, cfg2)
    with pytest.raises(TAError, match="does not match"):
        tr.load_base(d)
    tr.close()
    # an F16 tensor is refused like upload_bf16 does (base_loader.cpp:73)
    p = os.path.join(d, "model.safetensors")
    raw = open(p, "rb").read()
    open(p, "wb").write(raw.replace(b'"model.norm.weight":{"dtype":"BF16"', b'"model.norm.weight":{"dtype":"F16" ', 1))
    tr = _trainer(ctx, cfg)
    with pytest.raises(TAError, match="unsupported weight dtype"):
        tr.load_base(d)
    tr.close()


def test_resume_continues_bit_exactly(ctx, tmp_path):
    cfg, base, adapter, toks, tgts = _case()
    a = _trainer(ctx, cfg); rc.load_into_trainer(a, cfg, base, adapter)
    for s in range(4):
        a.step(toks[s], tgts[s], 2, lr=1e-3)
    want = a.download("lora.master"); want_m = a.download("lora.m"); want_c = a.download("centroid.acc")
    b = _trainer(ctx, cfg); rc.load_into_trainer(b, cfg, base, adapter)
    for s in range(2):
        b.step(toks[s], tgts[s], 2, lr=1e-3)
    ck = str(tmp_path / "step-2")
    b.save_checkpoint(ck)
    assert sorted(os.listdir(ck)) == ["adapter.json", "adapter.safetensors", "optimizer.safetensors", "train_state.json"]
    b.close()
    c = _trainer(ctx, cfg); rc.load_into_trainer(c, cfg, base, o.make_adapter(cfg, 16))   # fresh LoRA state
    c.resume(ck)
    assert (c.step_count, c.tokens_seen) == (2, 2 * 2 * 64)
    for s in range(2, 4):
        m = c.step(toks[s], tgts[s], 2, lr=1e-3)
    assert m.step == 4
    np.testing.assert_array_equal(c.download("lora.master"), want)
    np.testing.assert_array_equal(c.download("lora.m"), want_m)
    np.testing.assert_array_equal(c.download("centroid.acc"), want_c)
    a.close(); c.close()


def test_resume_from_reference_format_checkpoint(ctx, tmp_path):
    """No optimizer.safetensors (what the reference writes): masters = the BF16 file values, zero
    moments, counters from train_state.json; a wrong rank is refused by the adapter.json check."""
    from tensor_adapt_b200 import TAError
    cfg, base, adapter, toks, tgts = _case()
    a = _trainer(ctx, cfg); rc.load_into_trainer(a, cfg, base, adapter)
    a.step(toks[0], tgts[0], 2, lr=1e-3)
    ck = str(tmp_path / "ref-ck")
    a.save_checkpoint(ck, with_optimizer=False)
    master = a.download("lora.master")
    b = _trainer(ctx, cfg); rc.load_into_trainer(b, cfg, base, o.make_adapter(cfg, 16))
    b.resume(ck)
    assert (b.step_count, b.tokens_seen) == (1, 2 * 64)
    np.testing.assert_array_equal(b.download("lora.master"), o.bf16_round(master))
    assert not b.download("lora.m").any() and not b.download("lora.v").any()
    c = _trainer(ctx, cfg, rank=8, alpha=16.0)
    with pytest.raises(TAError, match="rank"):
        c.resume(ck)
    a.close(); b.close(); c.close()


@pytest.mark.parametrize("shards,tie", [(1, True), (2, False)])
def test_load_base_equals_reference_loader(ctx, tmp_path, shards, tie):
    """The unmodified BaseLoader::load (oracle/_ref/ref_harness load) and ta_trainer_load_base read the
    same directory: identical derived config, base_sha and BF16 bits of every tensor."""
    if not os.path.exists(rc.HARNESS):
        pytest.skip("oracle/_ref/ref_harness is not built")
    from tensor_adapt_b200.trainer import probe_base
    cfg, base, *_ = _case(tie)
    rng = np.random.default_rng(9)
    base["layers"][0]["k_w"] = (rng.standard_normal(base["layers"][0]["k_w"].shape) * 0.05).astype(np.float32)
    base["embed"] = (rng.standard_normal(base["embed"].shape) * 0.05).astype(np.float32)
    d, out = str(tmp_path / "hf"), str(tmp_path / "ref")
    o.write_hf_dir(d, cfg, base, shards=shards, f32_names={"model.layers.0.self_attn.k_proj.weight", "model.embed_tokens.weight"})
    rc.run_harness("load", d, out)
    ref_cfg = dict(l.split(None, 1) for l in open(os.path.join(out, "config.txt")).read().splitlines())
    mc, arch, sha = probe_base(d)
    assert arch == ref_cfg["arch_name"] and sha == ref_cfg["base_sha"]
    for k, v in (("vocab", mc.vocab), ("hidden", mc.hidden), ("layers", mc.layers), ("hq", mc.q_heads), ("hkv", mc.kv_heads),
                 ("hd", mc.head_dim), ("inter", mc.intermediate), ("tie", mc.tie_embeddings)):
        assert int(ref_cfg[k]) == v, k
    assert float(ref_cfg["eps"]) == pytest.approx(mc.rms_eps, rel=1e-6) and float(ref_cfg["theta"]) == pytest.approx(mc.rope_theta, rel=1e-6)
    tr = _trainer(ctx, cfg)
    tr.load_base(d)
    names = ["embed", "final_norm"] + ([] if tie else ["lm_head"]) + [f"l{l}.{k}" for l in range(cfg.layers) for k in rc.LAYER_KEYS]
    for n in names:
        ref = rc.bf16(os.path.join(out, n.replace(".", "_") + ".bin"))
        np.testing.assert_array_equal(tr.download(n).ravel(), ref, err_msg=n)
    tr.close()


def test_load_base_vs_reference_golden(ctx, tmp_path):
    """Committed fixture made by the reference's BaseLoader on the same seeded directory."""
    import hashlib
    import json
    from tensor_adapt_b200.trainer import probe_base
    g = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_load_tiny.json")))
    d = str(tmp_path / "hf")
    cfg, _ = rc.hf_case(d)
    mc, arch, sha = probe_base(d)
    c = g["config"]
    assert (arch, sha) == (c["arch_name"], c["base_sha"])
    assert [mc.vocab, mc.hidden, mc.layers, mc.q_heads, mc.kv_heads, mc.head_dim, mc.intermediate, mc.tie_embeddings] == \
        [int(c[k]) for k in ("vocab", "hidden", "layers", "hq", "hkv", "hd", "inter", "tie")]
    tr = _trainer(ctx, cfg)
    tr.load_base(d)
    for name, want in g["sha256_of_bf16_bytes"].items():
        tname = name.replace("_", ".", 1) if name[0] == "l" and name[1].isdigit() else name
        bits = o.bf16_bits(tr.download(tname).ravel()).astype("<u2").tobytes()
        assert hashlib.sha256(bits).hexdigest() == want, name
    tr.close()


def test_save_adapter_after_resume_merges_the_whole_run(ctx, tmp_path):
    """A run interrupted after its first snapshot and resumed ends with the same adapter.centroid as the
    uninterrupted run: the snapshot files already on disk come back into the merge list on resume."""
    cfg, base, adapter, toks, tgts = _case()

    def run(out, stop_after=None, resume_from=None):
        tr = _trainer(ctx, cfg); rc.load_into_trainer(tr, cfg, base, adapter if resume_from is None else o.make_adapter(cfg, 16))
        tr.output_dir, tr.checkpoint_every = str(out), 1
        first = 0
        if resume_from is not None:
            tr.resume(resume_from)
            first = tr.step_count
        for s in range(first, 4 if stop_after is None else stop_after):
            tr.step(toks[s], tgts[s], 2, lr=1e-3)          # writes centroids/step-N.centroid and step-N/ every step
        if stop_after is None:
            tr.save_adapter(str(out))
        tr.close()

    whole, parts = tmp_path / "whole", tmp_path / "parts"
    run(whole)
    run(parts, stop_after=2)
    run(parts, resume_from=str(parts / "step-2"))
    assert (parts / "adapter.centroid").read_bytes() == (whole / "adapter.centroid").read_bytes()
    assert o.read_merged_file(str(whole / "adapter.centroid")).shape[0] == 5       # 4 step snapshots + the final one


def test_resume_refuses_another_target_set(ctx, tmp_path):
    from tensor_adapt_b200 import TAError
    cfg, base, adapter, toks, tgts = _case()
    a = _trainer(ctx, cfg); rc.load_into_trainer(a, cfg, base, adapter)
    a.step(toks[0], tgts[0], 2, lr=1e-3)
    ck = str(tmp_path / "step-1")
    a.save_checkpoint(ck)
    a.close()
    b = _trainer(ctx, cfg, targets=7)                   # q/k/v only: other flat layout
    with pytest.raises(TAError, match="disagree on inject_o|another set of adapted projections"):
        b.resume(ck)
    b.close()
