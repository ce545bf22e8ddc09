"""Token stream in HBM: device-side next_batch + assistant-only masking against the oracle's
restatement of Dataset::next_batch (src/data/dataset.cpp:55-71) and of the masking state machine
(src/trainer/adapt_trainer.cu:145-182), including wrap-around, shards of the global batch, a directory
of .bin files and a training step drawn straight from the stream."""
import os

import numpy as np
import pytest
import torch

import refcase as rc
import ta_oracle as o

pytestmark = pytest.mark.gpu
IM_START, ASSISTANT, IM_END = 151644, 77091, 151645


def _chat_stream(n, seed, vocab=152000):
    """Random ids with chat turns sprinkled in: <|im_start|> role ... <|im_end|>, some turns by the assistant."""
    rng = np.random.default_rng(seed)
    t = rng.integers(0, 1000, n).astype(np.uint32)
    i = 0
    while i < n - 8:
        i += int(rng.integers(1, 40))
        if i >= n - 8:
            break
        t[i] = IM_START
        t[i + 1] = ASSISTANT if rng.random() < 0.5 else 872          # "user"
        j = i + 2 + int(rng.integers(0, 60))
        if j < n:
            t[j] = IM_END
        if rng.random() < 0.1 and i + 3 < n:
            t[i + 3] = ASSISTANT                                       # the word inside a turn is masked too
        i = j
    return t


def _ints(n):
    return torch.empty(n, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("n,B,T,batches", [(5000, 4, 256, 7), (300, 3, 128, 3), (70000, 2, 4096, 2), (1027, 5, 33, 9)])
def test_next_batch_and_mask_match_oracle(ctx, tmp_path, n, B, T, batches):
    from tensor_adapt_b200 import ptr
    from tensor_adapt_b200.trainer import Dataset
    toks = _chat_stream(n, seed=n)
    p = str(tmp_path / "train.bin"); toks.tofile(p)
    ds = Dataset(ctx, p)
    assert ds.total_tokens == n and ds.position == 0
    ids, tgt = _ints(B * T), _ints(B * T)
    pos = 0
    for k in range(batches):
        mask = k % 2 == 0
        ds.next_batch(B, T, ptr(ids), ptr(tgt), mask=mask)
        want_i, want_t, pos = o.next_batch(toks.astype(np.int64).astype(np.int32), pos, B, T)
        if mask:
            want_t = o.mask_targets(want_i, want_t, B, T)
        np.testing.assert_array_equal(ids.cpu().numpy(), want_i)
        np.testing.assert_array_equal(tgt.cpu().numpy(), want_t)
        assert ds.position == pos and ds.tokens_consumed == (k + 1) * B * T
    ds.close()


def test_shards_of_the_global_batch_and_directory_input(ctx, tmp_path):
    from tensor_adapt_b200 import ptr
    from tensor_adapt_b200.trainer import Dataset
    a, b = _chat_stream(3000, 1), _chat_stream(2500, 2)
    d = tmp_path / "data"; d.mkdir()
    b.tofile(str(d / "b.bin")); a.tofile(str(d / "a.bin")); (d / "notes.txt").write_text("ignored")
    toks = np.concatenate([a, b]).astype(np.int32)                   # files in sorted order
    B, T = 8, 128
    full_i, full_t, pos = o.next_batch(toks, 0, B, T)
    full_t = o.mask_targets(full_i, full_t, B, T)
    for rank, world in ((0, 2), (1, 2), (3, 4)):
        ds = Dataset(ctx, str(d))
        per = B // world
        ids, tgt = _ints(per * T), _ints(per * T)
        ds.next_batch(B, T, ptr(ids), ptr(tgt), first_seq=rank * per, n_seq=per)
        np.testing.assert_array_equal(ids.cpu().numpy(), full_i[rank * per * T:(rank + 1) * per * T])
        np.testing.assert_array_equal(tgt.cpu().numpy(), full_t[rank * per * T:(rank + 1) * per * T])
        assert ds.position == pos                                      # every rank advances by the GLOBAL batch
        ds.close()


def test_mask_targets_device_equals_host(ctx):
    from tensor_adapt_b200 import ptr, stream_ptr
    B, T = 6, 777
    ids = _chat_stream(B * T, 5).astype(np.int32)
    tgt = np.roll(ids, -1)
    want = o.mask_targets(ids, tgt.copy(), B, T)
    di, dt = torch.from_numpy(ids).cuda(), torch.from_numpy(tgt.copy()).cuda()
    ctx.call("ta_mask_targets_device", ptr(di), ptr(dt), B, T, stream_ptr())
    np.testing.assert_array_equal(dt.cpu().numpy(), want)


def test_step_from_the_stream_equals_step_on_host_arrays(ctx, tmp_path):
    from tensor_adapt_b200 import TAError
    from tensor_adapt_b200.trainer import AdaptTrainer, AdapterConfig, Dataset
    cfg = rc.tiny_cfg(hidden=128, hq=2, hkv=1, hd=64, inter=256, vocab=152064, layers=1)
    B, T = 2, 128
    base, adapter, _, _ = rc.make_case(cfg, B, T, 16, seed=3, std=0.05, b_std=0.05)
    toks = _chat_stream(900, 8)
    p = str(tmp_path / "t.bin"); toks.tofile(p)
    ac = AdapterConfig.defaults(rank=16, alpha=32.0, targets=15, lr=1e-3)
    a = AdaptTrainer(ctx, rc.model_config(cfg), ac, B, T); rc.load_into_trainer(a, cfg, base, adapter)
    b = AdaptTrainer(ctx, rc.model_config(cfg), ac, B, T); rc.load_into_trainer(b, cfg, base, adapter)
    ds = Dataset(ctx, p)
    pos = 0
    for s in range(4):                                                  # 4 x 256 tokens wrap the 900-token stream
        ma = a.step_dataset(ds, B, lr=1e-3)
        wi, wt, pos = o.next_batch(toks.astype(np.int32), pos, B, T)
        mb = b.step(wi, o.mask_targets(wi, wt, B, T), B, lr=1e-3)
        assert ma.loss == mb.loss and ma.grad_norm_raw == mb.grad_norm_raw and ma.tokens_consumed == mb.tokens_consumed
    np.testing.assert_array_equal(a.download("lora.master"), b.download("lora.master"))
    with pytest.raises(TAError, match="path not found"):
        Dataset(ctx, str(tmp_path / "missing"))
    e = tmp_path / "empty"; e.mkdir()
    with pytest.raises(TAError, match="no .bin files"):
        Dataset(ctx, str(e))
    ds.close(); a.close(); b.close()
