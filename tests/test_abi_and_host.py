"""CPU-only checks of the boundary: the shared library loads without a GPU, exports exactly the
entry points include/tensor_adapt_b200.h declares, fails loudly (no fallback) when no sm_100 device is
present, and its host-side logic (cosine schedule, target masking, Kaiming hash) matches the oracle."""
import ctypes
import os
import re

import numpy as np
import pytest

import ta_oracle as o

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    txt = open(os.path.join(ROOT, "include", "tensor_adapt_b200.h")).read()
    txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
    return sorted(set(re.findall(r"\b(ta_[a-z0-9_]+)\s*\(", txt)))


def test_library_exports_every_declared_symbol():
    import tensor_adapt_b200 as ta
    declared = header_symbols()
    assert len(declared) >= 45
    missing = [s for s in declared if not hasattr(ta.lib, s)]
    assert not missing, f"declared in the header but not exported: {missing}"
    unbound = sorted(set(declared) - set(ta.exported_symbols()))
    assert not unbound, f"declared in the header but not bound in _lib.py: {unbound}"
    undeclared = sorted(set(ta.exported_symbols()) - set(declared))
    assert not undeclared, f"bound in _lib.py but not declared in the header: {undeclared}"


@pytest.mark.parametrize("compiler,flags", [("gcc", ["-std=c99", "-x", "c"]), ("g++", ["-std=c++17", "-x", "c++"])])
def test_header_compiles_as_plain_c_and_cpp(compiler, flags, tmp_path):
    """The boundary is a C ABI: the header must stand alone (no CUDA headers) for a C99 and a C++ compiler,
    and a translation unit that takes the address of an entry point must compile against it."""
    import shutil
    import subprocess
    if not shutil.which(compiler):
        pytest.skip(f"{compiler} not installed")
    src = tmp_path / "use_header.c"
    src.write_text('#include "tensor_adapt_b200.h"\n'
                   'int probe(void) { ta_ctx* c = 0; int s = 0; return ta_device_status(c, &s) + TA_ERR_INVALID; }\n'
                   'int (*p_batch)(ta_dataset*, int, int, int, int, int*, int*, int, void*) = ta_dataset_next_batch;\n')
    r = subprocess.run([compiler, *flags, "-Wall", "-Werror", "-pedantic", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), str(src)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_every_entry_point_cites_the_reference():
    txt = open(os.path.join(ROOT, "include", "tensor_adapt_b200.h")).read()
    # each declaration block is preceded by a comment naming a reference file:line
    assert len(re.findall(r"\.(?:cu|cpp|hpp):\d+", txt)) >= 40


def test_no_silent_fallback_without_gpu():
    import torch
    import tensor_adapt_b200 as ta
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(ta.TAError):
        ta.Context(0)


def test_cosine_schedule_matches_reference_formula():
    import tensor_adapt_b200 as ta
    for warm, total in ((1, 10), (100, 1000), (200, 6103)):
        for step in (0, 1, warm - 1, warm, warm + 1, total // 2, total - 1, total, total + 50):
            if step < 0:
                continue
            got = ta.lib.ta_cosine_lr(2e-4, warm, total, step, 0.1)
            assert abs(got - o.cosine_lr(2e-4, warm, total, step)) <= 1e-10 + 1e-6 * got


def test_mask_targets_state_machine():
    import tensor_adapt_b200 as ta
    rng = np.random.default_rng(0)
    B, T = 3, 64
    ids = rng.integers(0, 1000, B * T).astype(np.int32)
    # plant chat turns: <|im_start|> assistant ... <|im_end|>, a user turn, an unterminated turn, a
    # start token in the last position of a row
    ids[5], ids[6], ids[20] = o.IM_START, o.ASSISTANT, o.IM_END
    ids[30], ids[31], ids[40] = o.IM_START, 872, o.IM_END
    ids[T + 3], ids[T + 4] = o.IM_START, o.ASSISTANT
    ids[2 * T - 1] = o.IM_START
    tgt = rng.integers(0, 1000, B * T).astype(np.int32)
    ref = o.mask_targets(ids, tgt, B, T)
    got = tgt.copy()
    ta.lib.ta_mask_targets(ids.ctypes.data_as(ctypes.c_void_p), got.ctypes.data_as(ctypes.c_void_p), B, T)
    assert np.array_equal(got, ref)
    assert (ref[7:21] >= 0).all() and ref[5] == -1 and ref[6] == -1
    # <|im_end|> is trained on even when it closes a non-assistant turn (adapt_trainer.cu:170-176)
    assert ref[40] >= 0 and (np.delete(ref[21:T], 40 - 21) == -1).all()


def test_kaiming_hash_init_bits():
    import tensor_adapt_b200 as ta
    for in_dim, rank in ((896, 16), (64, 2), (3584, 64)):
        out = np.empty(in_dim * rank, dtype=np.float32)
        ta.lib.ta_kaiming_init_host(out.ctypes.data_as(ctypes.c_void_p), in_dim, rank, 0x1234)
        ref = o.kaiming_init(in_dim, rank).ravel()
        assert np.array_equal(out, ref)
        assert np.abs(ref).max() <= np.sqrt(1.0 / in_dim) + 1e-9


def test_shard_ranges():
    from tensor_adapt_b200.dp import shard_batch, shard_range
    assert [shard_range(32, r, 8) for r in range(8)] == [(4 * r, 4 * r + 4) for r in range(8)]
    with pytest.raises(ValueError):
        shard_range(10, 0, 4)
    tok = np.arange(8 * 4); tgt = tok + 1
    a, b, n = shard_batch(tok, tgt, 8, 4, 1, 2)
    assert n == 4 and a[0] == 16 and b[-1] == 32


def test_reference_arm_of_bench_does_not_load_the_product_library():
    """`bench.py --impl reference` must time the reference alone: the process prints its one JSON line (a
    measurement on a GPU box, an `unavailable` line elsewhere) without ever importing the CUDA package."""
    import json
    import subprocess
    import sys
    code = ("import sys, runpy\n"
            f"sys.argv = ['bench.py', '--impl', 'reference', '--steps', '1', '--warmup', '0', '--config', 'qwen2-0.5b']\n"
            f"runpy.run_path({os.path.join(ROOT, 'bench.py')!r}, run_name='__main__')\n"
            "assert not [m for m in sys.modules if m.startswith('tensor_adapt_b200')], 'product package imported'\n")
    import torch
    if torch.cuda.is_available():
        pytest.skip("on a GPU box this would run the reference's full step; the GPU tests cover it")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert line["impl"] == "reference" and ("unavailable" in line or line["value"] > 0)


def test_shim_built_reference_tools_fail_loudly_without_a_gpu(tmp_path):
    """The reference's unmodified tools linked on the shim have no CPU path either: without an sm_100 device they
    exit with the reference's own error convention (message on stderr, exit code 1), they do not fall back."""
    import struct
    import subprocess
    import torch
    tool = os.path.join(ROOT, "oracle", "_ref", "shim", "centroid-merge")
    if not os.path.exists(tool):
        pytest.skip("shim tools not built (needs the reference checkout)")
    if torch.cuda.is_available():
        pytest.skip("a GPU is present; tests/test_gpu_shim_tools.py covers the tools")
    d = tmp_path / "snaps"; d.mkdir()
    for i in range(3):
        (d / f"step-{i}.centroid").write_bytes(struct.pack("<i", 8) + np.arange(8, dtype="<f4").tobytes() + struct.pack("<f", 1.0))
    r = subprocess.run([tool, str(d), "--out", str(tmp_path / "out.centroid"), "--clusters", "2"], capture_output=True, text=True)
    assert r.returncode == 1 and "error:" in r.stderr and not (tmp_path / "out.centroid").exists()
