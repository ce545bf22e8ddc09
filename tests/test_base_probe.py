"""Host side of real-weight loading (no GPU): config.json with the reference's defaults, shard
discovery, base_sha and header validation errors of ta_base_probe."""
import json
import os
import struct

import numpy as np
import pytest

import refcase as rc
import ta_oracle as o


def _tiny():
    cfg = rc.tiny_cfg(hidden=128, hq=2, hkv=1, hd=64, inter=256, vocab=320, layers=2)
    return cfg, o.make_base(cfg, np.random.default_rng(3))


@pytest.mark.parametrize("shards", [1, 3])
def test_probe_reads_config_and_sha(tmp_path, shards):
    from tensor_adapt_b200.trainer import probe_base
    cfg, base = _tiny()
    d = str(tmp_path / "m")
    o.write_hf_dir(d, cfg, base, shards=shards)
    mc, arch, sha = probe_base(d)
    assert (mc.vocab, mc.hidden, mc.layers, mc.q_heads, mc.kv_heads, mc.head_dim, mc.intermediate) == (320, 128, 2, 2, 1, 64, 256)
    assert mc.rms_eps == pytest.approx(1e-6) and mc.rope_theta == pytest.approx(1e6)
    assert mc.tie_embeddings == 1 and arch == "qwen2"
    assert sha == o.base_sha(d)                      # SHA-256 of the "name:size;" listing (base_loader.cpp:30-52)


def test_probe_defaults_and_untied_head(tmp_path):
    from tensor_adapt_b200.trainer import probe_base
    cfg, base = _tiny()
    cfg.tie = False
    base["lm_head"] = base["embed"].copy()
    d = str(tmp_path / "m")
    o.write_hf_dir(d, cfg, base)
    with open(os.path.join(d, "config.json"), "w") as f:     # only model_type: every size falls back to its default
        json.dump({"model_type": "qwen2", "num_attention_heads": 16}, f)
    mc, arch, _ = probe_base(d)
    assert (mc.vocab, mc.hidden, mc.layers, mc.q_heads, mc.kv_heads, mc.intermediate) == (32000, 4096, 32, 16, 16, 11008)
    assert mc.head_dim == 256 and mc.rms_eps == pytest.approx(1e-5) and mc.rope_theta == pytest.approx(10000.0)
    assert mc.tie_embeddings == 0                            # lm_head.weight is present in the shards


def test_model_safetensors_wins_over_other_shards(tmp_path):
    """WeightMap::open (weight_map.cpp:40-44): <dir>/model.safetensors alone is read when it exists -
    a second file that would otherwise be a duplicate-name error is ignored - but base_sha lists both."""
    from tensor_adapt_b200.trainer import probe_base
    cfg, base = _tiny()
    d = str(tmp_path / "m")
    o.write_hf_dir(d, cfg, base)
    o.write_safetensors_file(os.path.join(d, "extra.safetensors"), {"model.norm.weight": base["final_norm"]})
    _, _, sha = probe_base(d)
    assert sha == o.base_sha(d)


def test_probe_errors(tmp_path):
    from tensor_adapt_b200 import TAError
    from tensor_adapt_b200.trainer import probe_base
    cfg, base = _tiny()
    with pytest.raises(TAError, match="does not exist"):
        probe_base(str(tmp_path / "nope"))
    d = str(tmp_path / "empty"); os.makedirs(d)
    with pytest.raises(TAError, match="no .safetensors files"):
        probe_base(d)
    d = str(tmp_path / "dup")
    o.write_hf_dir(d, cfg, base, shards=2)
    o.write_safetensors_file(os.path.join(d, "zz.safetensors"), {"model.norm.weight": base["final_norm"]})
    with pytest.raises(TAError, match="duplicate tensor name"):
        probe_base(d)
    d = str(tmp_path / "arch")
    o.write_hf_dir(d, cfg, base, model_type="mamba")
    with pytest.raises(TAError, match="unknown architecture: mamba"):
        probe_base(d)
    mc, arch, _ = probe_base(d, arch_hint="qwen2")            # the hint overrides model_type (base_loader.cpp:21-28)
    assert arch == "mamba" and mc.hidden == 128
    d = str(tmp_path / "bad")
    o.write_hf_dir(d, cfg, base)
    p = os.path.join(d, "model.safetensors")
    raw = open(p, "rb").read()
    for mutate, msg in (
            (lambda b: struct.pack("<Q", 0) + b[8:], "header length is zero"),
            (lambda b: struct.pack("<Q", len(b)) + b[8:], "exceeds file size"),
            (lambda b: b[:8] + b"[" + b[9:], "JSON parse error"),
            (lambda b: b[:len(b) - 64], "exceeds file size")):
        open(p, "wb").write(mutate(raw))
        with pytest.raises(TAError, match=msg):
            probe_base(d)


def test_probe_survives_corrupted_headers(tmp_path):
    """Byte-level corruption of a valid safetensors header (flipped bytes, truncations, random lengths) must
    end in a clean success or a TAError - never a crash or a hang: the header is untrusted input."""
    from tensor_adapt_b200 import TAError
    from tensor_adapt_b200.trainer import probe_base
    cfg, base = _tiny()
    d = str(tmp_path / "m")
    o.write_hf_dir(d, cfg, base)
    p = os.path.join(d, "model.safetensors")
    raw = open(p, "rb").read()
    hlen = struct.unpack("<Q", raw[:8])[0]
    rng = np.random.default_rng(0)
    outcomes = {"ok": 0, "err": 0}
    for trial in range(300):
        b = bytearray(raw[:8 + hlen + 4096])           # header + a little data is enough for the parser
        kind = trial % 4
        if kind == 0:                                   # flip a few header bytes
            for _ in range(int(rng.integers(1, 6))):
                b[8 + int(rng.integers(0, hlen))] = int(rng.integers(0, 256))
        elif kind == 1:                                 # truncate inside the header
            b = b[:8 + int(rng.integers(0, hlen))]
        elif kind == 2:                                 # lie about the header length
            b[:8] = struct.pack("<Q", int(rng.integers(0, 2 * len(b))))
        else:                                           # splice structural characters in
            pos = 8 + int(rng.integers(0, hlen))
            b[pos:pos] = bytes(rng.choice(list(b'{}[]",:\\'), size=int(rng.integers(1, 8))).tolist())
        open(p, "wb").write(bytes(b))
        try:
            probe_base(d)
            outcomes["ok"] += 1
        except TAError:
            outcomes["err"] += 1
    assert outcomes["err"] > 100 and outcomes["ok"] + outcomes["err"] == 300
