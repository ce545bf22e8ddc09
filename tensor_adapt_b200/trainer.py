"""Host-side mirror of the reference's trainer interface over the C ABI.

`AdaptTrainer` carries the names of tensor::trainer::AdaptTrainer (include/tensor/trainer/
adapt_trainer.hpp:48-78): step(), done(), save_checkpoint(), save_adapter(); `AdapterConfig` /
`ModelConfig` / `StepMetrics` are the C structs of include/tensor_adapt_b200.h.  All compute happens
in libtensor_adapt_b200.so; NumPy is used only to move test data in and out.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_long, c_void_p
from typing import Optional

import numpy as np

from ._lib import Context, TAError, lib  # noqa: F401

TARGET_BITS = {"q": 1, "k": 2, "v": 4, "o": 8, "gate": 16, "up": 32, "down": 64}
TARGETS_QKVO = 15
TARGETS_ALL = 127


class ModelConfig(ctypes.Structure):
    _fields_ = [("vocab", c_int), ("hidden", c_int), ("layers", c_int), ("q_heads", c_int), ("kv_heads", c_int),
                ("head_dim", c_int), ("intermediate", c_int), ("rms_eps", c_float), ("rope_theta", c_float),
                ("tie_embeddings", c_int)]


class AdapterConfig(ctypes.Structure):
    _fields_ = [("rank", c_int), ("alpha", c_float), ("targets", c_int), ("lr", c_float), ("grad_clip", c_float),
                ("warmup_steps", c_int), ("beta1", c_float), ("beta2", c_float), ("eps", c_float),
                ("weight_decay", c_float), ("centroid_modes", c_int)]

    @classmethod
    def defaults(cls, rank=16, alpha=16.0, targets=TARGETS_QKVO, lr=2e-4, grad_clip=1.0, warmup_steps=200, beta1=0.9,
                 beta2=0.999, eps=1e-8, weight_decay=0.0, centroid_modes=1):
        """Defaults of include/tensor/adapter/adapter_config.hpp:29-53."""
        return cls(rank, alpha, targets, lr, grad_clip, warmup_steps, beta1, beta2, eps, weight_decay, centroid_modes)


class StepMetrics(ctypes.Structure):
    _fields_ = [("step", c_long), ("tokens_consumed", c_long), ("loss", c_float), ("learning_rate", c_float),
                ("grad_norm", c_float), ("grad_norm_raw", c_float)]


QWEN2 = {
    # shapes of Qwen2-0.5B / 1.5B / 7B
    "qwen2-0.5b": ModelConfig(151936, 896, 24, 14, 2, 64, 4864, 1e-6, 1e6, 1),
    "qwen2-1.5b": ModelConfig(151936, 1536, 28, 12, 2, 128, 8960, 1e-6, 1e6, 1),
    "qwen2-7b": ModelConfig(152064, 3584, 28, 28, 4, 128, 18944, 1e-6, 1e6, 0),
}


def probe_base(directory: str, arch_hint: str = ""):
    """(ModelConfig, model_type, base_sha) of a Hugging Face model directory, as BaseLoader::load derives
    them (src/base/base_loader.cpp:90-110); host only."""
    mc = ModelConfig()
    arch, sha, err = ctypes.create_string_buffer(64), ctypes.create_string_buffer(65), ctypes.create_string_buffer(512)
    rc = lib.ta_base_probe(directory.encode(), arch_hint.encode(), ctypes.byref(mc), arch, 64, sha, 65, err, 512)
    if rc != 0:
        raise TAError(rc, err.value.decode(errors="replace"))
    return mc, arch.value.decode(), sha.value.decode()


class Dataset:
    """data::Dataset (include/tensor/data/dataset.hpp) with the token stream resident in HBM."""

    def __init__(self, ctx: Context, path: str):
        self.ctx, h = ctx, c_void_p()
        ctx.call("ta_dataset_load", path.encode(), ctypes.byref(h))
        self.h = h

    def _info(self):
        a, b, c = c_long(0), c_long(0), c_long(0)
        lib.ta_dataset_info(self.h, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c))
        return a.value, b.value, c.value

    total_tokens = property(lambda self: self._info()[0])
    position = property(lambda self: self._info()[1])
    tokens_consumed = property(lambda self: self._info()[2])

    def seek(self, position: int, tokens_consumed: int = 0) -> None:
        lib.ta_dataset_seek(self.h, position, tokens_consumed)

    def next_batch(self, B: int, T: int, ids_ptr, targets_ptr, first_seq: int = 0, n_seq: int = -1, mask: bool = True,
                   stream=None) -> None:
        """Fills device arrays (pointers) with sequences [first_seq, first_seq+n_seq) of the next global batch."""
        rc = lib.ta_dataset_next_batch(self.h, B, T, first_seq, B - first_seq if n_seq < 0 else n_seq, ids_ptr, targets_ptr,
                                       int(mask), stream)
        if rc != 0:
            raise TAError(rc, (lib.ta_last_error(self.ctx.h) or b"").decode())

    def close(self) -> None:
        if self.h:
            lib.ta_dataset_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return ((u + (((u >> 16) & 1) + np.uint32(0x7FFF))) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


class _CudaView:
    """Zero-copy view of library-owned device memory for torch.as_tensor (CUDA array interface)."""

    def __init__(self, ptr: int, n: int, typestr: str):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 2}


class AdaptTrainer:
    def __init__(self, ctx: Context, model: ModelConfig, adapter: AdapterConfig, micro_batch: int, seq_len: int,
                 stream: Optional[int] = None, total_tokens: int = 0, output_dir: Optional[str] = None,
                 domain: str = "", checkpoint_every: int = 1000):
        self.ctx, self.model, self.adapter = ctx, model, adapter
        self.seq_len, self.micro_batch = seq_len, micro_batch
        h = c_void_p()
        rc = lib.ta_trainer_create(ctx.h, ctypes.byref(model), ctypes.byref(adapter), micro_batch, seq_len,
                                   c_void_p(stream or 0), ctypes.byref(h))
        if rc:
            raise TAError(rc, (lib.ta_last_error(ctx.h) or b"").decode())
        self.h = h
        self.output_dir, self.domain, self.checkpoint_every = output_dir, domain, checkpoint_every
        self.total_tokens = total_tokens
        self.tokens_seen = 0
        self.step_count = 0

    # ── plumbing ────────────────────────────────────────────────────────────
    def _call(self, name, *args):
        rc = getattr(lib, name)(self.h, *args)
        if rc:
            raise TAError(rc, (lib.ta_last_error(self.ctx.h) or b"").decode())

    def tensor(self, name: str):
        p = c_void_p(); r = c_long(); c = c_long(); pitch = c_long(); dt = c_int()
        self._call("ta_trainer_tensor", name.encode(), ctypes.byref(p), ctypes.byref(r), ctypes.byref(c),
                   ctypes.byref(pitch), ctypes.byref(dt))
        return p.value, r.value, c.value, pitch.value, dt.value

    def upload(self, name: str, a: np.ndarray) -> None:
        p, r, c, pitch, dt = self.tensor(name)
        a = np.asarray(a, dtype=np.float32).reshape(r, c)
        buf = np.zeros((r, pitch), dtype=np.float32)
        buf[:, :c] = a
        host = f32_to_bf16_bits(buf) if dt == 1 else buf
        host = np.ascontiguousarray(host)
        rc = lib.ta_memcpy_h2d(c_void_p(p), host.ctypes.data_as(c_void_p), host.nbytes)
        if rc:
            raise TAError(rc, f"upload {name}")

    def download(self, name: str) -> np.ndarray:
        p, r, c, pitch, dt = self.tensor(name)
        host = np.empty((r, pitch), dtype=np.uint16 if dt == 1 else np.float32)
        rc = lib.ta_memcpy_d2h(host.ctypes.data_as(c_void_p), c_void_p(p), host.nbytes)
        if rc:
            raise TAError(rc, f"download {name}")
        out = bf16_bits_to_f32(host) if dt == 1 else host
        return np.ascontiguousarray(out.reshape(r, pitch)[:, :c])

    def torch_view(self, name: str):
        """torch tensor aliasing a flat FP32 array of the trainer (e.g. "lora.grad" for the
        data-parallel all-reduce)."""
        import torch
        p, r, c, pitch, dt = self.tensor(name)
        assert dt == 0 and r == 1
        return torch.as_tensor(_CudaView(p, c, "<f4"), device=f"cuda:{self.ctx.device}")

    def torch_tensor(self, name: str):
        """Zero-copy 2-D torch view [rows, cols] (row pitch respected) of any named tensor, FP32 or BF16."""
        import torch
        p, r, c, pitch, dt = self.tensor(name)
        flat = torch.as_tensor(_CudaView(p, r * pitch, "<f4" if dt == 0 else "<i2"), device=f"cuda:{self.ctx.device}")
        if dt == 1:
            flat = flat.view(torch.bfloat16)
        return flat.view(r, pitch)[:, :c]

    # ── model state ─────────────────────────────────────────────────────────
    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        self._call("ta_trainer_init_random", seed, std)

    def sync_working(self) -> None:
        self._call("ta_trainer_sync_working")

    def load_base(self, directory: str, arch_hint: str = "") -> None:
        """BaseLoader::load (src/base/base_loader.cpp:80-170): config.json + safetensors shards of a
        Hugging Face checkpoint into the frozen-weight arena."""
        self._call("ta_trainer_load_base", directory.encode(), arch_hint.encode())

    def save_optimizer(self, directory: str) -> None:
        self._call("ta_trainer_save_optimizer", directory.encode())

    def resume(self, directory: str) -> None:
        """Restore masters, AdamW moments, centroid sums, step and token counters from a checkpoint."""
        self._call("ta_trainer_resume", directory.encode())
        st, tk = c_long(0), c_long(0)
        self._call("ta_trainer_counters", ctypes.byref(st), ctypes.byref(tk))
        self.step_count, self.tokens_seen = st.value, tk.value

    def set_meta(self, arch_name: str, base_sha: str) -> None:
        self._call("ta_trainer_set_meta", arch_name.encode(), base_sha.encode())

    # ── the step ────────────────────────────────────────────────────────────
    @staticmethod
    def _ids(a):
        if hasattr(a, "data_ptr"):          # torch tensor (pinned host or device)
            return c_void_p(a.data_ptr()), (0 if a.is_cuda else 1), a
        a = np.ascontiguousarray(a, dtype=np.int32)
        return a.ctypes.data_as(c_void_p), 1, a

    def zero_grad(self) -> None:
        self._call("ta_trainer_zero_grad")

    def forward_backward(self, tokens, targets, B: int, global_tokens: int = 0) -> None:
        tp, host, _k1 = self._ids(tokens)
        gp, _, _k2 = self._ids(targets)
        self._call("ta_trainer_forward_backward", tp, gp, B, self.seq_len, global_tokens, host)

    def optimizer_step(self, lr: float = -1.0, total_steps: int = 0) -> StepMetrics:
        m = StepMetrics()
        self._call("ta_trainer_optimizer_step", lr, total_steps, ctypes.byref(m))
        self.step_count = m.step
        self.tokens_seen = m.tokens_consumed
        return m

    def step(self, tokens, targets, B: int, lr: float = -1.0, total_steps: int = 0) -> StepMetrics:
        """AdaptTrainer::step on caller-provided ids; periodic checkpoint as adapt_trainer.cu:265-270."""
        tp, host, _k1 = self._ids(tokens)
        gp, _, _k2 = self._ids(targets)
        m = StepMetrics()
        self._call("ta_trainer_step", tp, gp, B, self.seq_len, lr, total_steps, host, ctypes.byref(m))
        self.step_count = m.step
        self.tokens_seen = m.tokens_consumed
        if self.output_dir and self.checkpoint_every and m.step % self.checkpoint_every == 0:
            self.write_snapshot(m.step)
            self.save_checkpoint(os.path.join(self.output_dir, f"step-{m.step}"))
        return m

    def step_dataset(self, ds: "Dataset", B: int, mask: bool = True, lr: float = -1.0, total_steps: int = 0) -> StepMetrics:
        """AdaptTrainer::step with the batch drawn and masked on the device (no host arrays involved)."""
        m = StepMetrics()
        self._call("ta_trainer_step_dataset", ds.h, B, int(mask), lr, total_steps, ctypes.byref(m))
        self.step_count, self.tokens_seen = m.step, m.tokens_consumed
        return m

    def done(self) -> bool:
        return self.tokens_seen >= self.total_tokens

    # ── artefacts ───────────────────────────────────────────────────────────
    def write_snapshot(self, step: int, mode: int = 0):
        D = self.model.hidden
        cen = np.zeros(D, dtype=np.float32); w = c_float(0)
        path = None
        if self.output_dir:
            d = os.path.join(self.output_dir, "centroids")
            os.makedirs(d, exist_ok=True)
            path = os.path.join(d, f"step-{step}.centroid").encode()
        self._call("ta_trainer_write_snapshot", mode, path, cen.ctypes.data_as(c_void_p), ctypes.byref(w))
        return cen, w.value

    def write_snapshot_bank(self, path: Optional[str] = None):
        """Per-layer centroid bank (AdapterConfig.centroid_modes bit 2): (centroids [layers, hidden], weights [layers]);
        `path` receives one reference-layout snapshot record per layer."""
        L, D = self.model.layers, self.model.hidden
        cen = np.zeros((L, D), dtype=np.float32); w = np.zeros(L, dtype=np.float32); n = c_int(0)
        self._call("ta_trainer_write_snapshot_bank", path.encode() if path else None, cen.ctypes.data_as(c_void_p),
                   w.ctypes.data_as(c_void_p), ctypes.byref(n))
        return cen, w

    def save_checkpoint(self, directory: str, with_optimizer: bool = True) -> None:
        """AdapterWriter::save_checkpoint files, plus optimizer.safetensors (what `resume` needs for an
        exact continuation)."""
        self._call("ta_trainer_save_checkpoint", directory.encode(), self.domain.encode(), self.step_count,
                   self.tokens_seen, 0)
        if with_optimizer:
            self.save_optimizer(directory)

    def save_adapter(self, directory: str, k: int = 16) -> None:
        """AdaptTrainer::save_adapter (adapt_trainer.cu:319-330): snapshot, k-means merge of the
        in-memory snapshots into adapter.centroid, final adapter files."""
        self.write_snapshot(self.step_count)
        os.makedirs(directory, exist_ok=True)
        passes = c_int(0)
        self._call("ta_trainer_merge_snapshots", k, os.path.join(directory, "adapter.centroid").encode(),
                   ctypes.byref(passes))
        self._call("ta_trainer_save_checkpoint", directory.encode(), self.domain.encode(), self.step_count,
                   self.tokens_seen, 1)

    def close(self) -> None:
        if self.h:
            lib.ta_trainer_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def centroid_merge_ranked(ctx: Context, snapshot_dir: str, out_path: str, k: int = 16, seed: int = 0, plusplus: bool = True,
                          rank_by_mass: bool = True):
    """Seeded k-means++ merge with the bank ordered by gradient mass (README.md:73-79; extension)."""
    n, passes = c_int(0), c_int(0)
    ctx.call("ta_centroid_merge_dir_ex", snapshot_dir.encode(), out_path.encode(), k, int(plusplus), seed, int(rank_by_mass),
             ctypes.byref(n), ctypes.byref(passes))
    return n.value, passes.value


def centroid_merge(ctx: Context, snapshot_dir: str, out_path: str, k: int = 16):
    """CentroidMerge::run (include/tensor/centroid/centroid_merge.hpp:12-19) on the GPU."""
    n = c_int(0); passes = c_int(0)
    ctx.call("ta_centroid_merge_dir", snapshot_dir.encode(), out_path.encode(), k, ctypes.byref(n), ctypes.byref(passes))
    return n.value, passes.value
