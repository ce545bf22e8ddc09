"""ctypes binding of libtensor_adapt_b200.so (the C ABI declared in include/tensor_adapt_b200.h).

The library is the product; this module only loads it and checks return codes.  There is no
Python or CPU fallback: if the shared library is missing or fails to load, importing raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_long, c_size_t, c_void_p

_PKG = os.path.dirname(os.path.abspath(__file__))
# TENSOR_ADAPT_B200_LIB points at another build of the same library (e.g. an experimental one beside the installed one)
LIB_PATH = os.environ.get("TENSOR_ADAPT_B200_LIB") or os.path.join(_PKG, "libtensor_adapt_b200.so")

TA_OK = 0
ERR_NAMES = {-1: "TA_ERR_INVALID", -2: "TA_ERR_CUDA", -3: "TA_ERR_UNSUPPORTED", -4: "TA_ERR_DEVICE_TIMEOUT",
             -5: "TA_ERR_NOMEM", -6: "TA_ERR_IO"}


class TAError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"{ERR_NAMES.get(code, code)}: {msg}")
        self.code = code


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is not built. Run `python -c 'import __graft_entry__ as g; g.build()'` "
            "(or `make -C tensor_adapt_b200`); there is no fallback implementation.")
    # torch first, so that libcudart / libnccl resolve to the copies torch already mapped
    try:
        import torch  # noqa: F401
    except Exception:
        pass
    return ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)


lib = _load()

P = c_void_p
_PROTOS = {
    "ta_ctx_create": (c_int, [c_int, POINTER(c_void_p)]),
    "ta_ctx_destroy": (c_int, [P]),
    "ta_ctx_set_workspace": (c_int, [P, P, c_size_t]),
    "ta_last_error": (c_char_p, [P]),
    "ta_device_status": (c_int, [P, POINTER(c_int)]),
    "ta_launch_count": (c_long, [P]),
    "ta_selftest_bounded_wait": (c_int, [P, c_int, POINTER(c_int), POINTER(c_int), P]),
    "ta_ctx_set_gemm_tuning": (c_int, [P, c_int, c_int, c_int]),
    "ta_ctx_set_gemm_raster": (c_int, [P, c_int, c_int]),
    "ta_profile_enable": (c_int, [P, c_int]),
    "ta_profile_read": (c_int, [P, c_int, POINTER(c_long), POINTER(ctypes.c_double), POINTER(ctypes.c_double)]),
    "ta_rms_norm_fwd": (c_int, [P, P, P, P, P, c_int, c_int, c_float, P]),
    "ta_rms_norm_bwd": (c_int, [P, P, P, P, P, P, P, c_int, c_int, P]),
    "ta_rope": (c_int, [P, P, c_int, P, c_int, c_int, c_int, c_int, c_float, c_int, P]),
    "ta_silu_mul_fwd": (c_int, [P, P, P, P, c_long, P]),
    "ta_silu_mul_bwd": (c_int, [P, P, P, P, P, P, c_long, P]),
    "ta_cross_entropy_fwd": (c_int, [P, P, P, P, P, c_int, c_int, c_float, P]),
    "ta_lmhead_ce_fwd_bwd": (c_int, [P, P, P, P, P, P, c_int, c_int, c_int, c_float, P, c_int, P]),
    "ta_embed_fwd": (c_int, [P, P, P, P, c_int, c_int, P]),
    "ta_add_bias": (c_int, [P, P, P, c_long, c_int, P]),
    "ta_add_inplace": (c_int, [P, P, P, c_long, P]),
    "ta_lora_add": (c_int, [P, P, P, c_float, c_long, P]),
    "ta_cast_bf16_to_f32": (c_int, [P, P, P, c_long, P]),
    "ta_cast_f32_to_bf16": (c_int, [P, P, P, c_long, P]),
    "ta_gemm_bf16": (c_int, [P, c_int, c_int, c_int, c_float, P, c_long, c_int, P, c_long, c_int, P, P, P, c_long, P]),
    "ta_swiglu_proj_fwd": (c_int, [P, P, P, P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_float, P]),
    "ta_swiglu_down_bwd": (c_int, [P, P, P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, P]),
    "ta_trainer_set_option": (c_int, [P, c_char_p, c_int]),
    "ta_lora_linear_fwd": (c_int, [P, P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_float, P]),
    "ta_lora_linear_bwd": (c_int, [P, P, P, P, P, P, P, c_int, P, P, c_int, c_int, c_int, c_int, c_float, P]),
    "ta_flash_attn_fwd": (c_int, [P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, P]),
    "ta_flash_attn_bwd": (c_int, [P, P, P, P, P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, P]),
    "ta_sum_sq_into": (c_int, [P, P, P, c_long, P]),
    "ta_adamw_step": (c_int, [P, P, P, P, P, P, c_long, c_float, c_float, c_float, c_float, c_float, c_int, P]),
    "ta_gradnorm_clip_adamw": (c_int, [P, P, P, P, P, P, c_long, c_float, c_float, c_float, c_float, c_float, c_int,
                                       c_float, P, c_int, P]),
    "ta_centroid_accumulate": (c_int, [P, c_int, P, P, c_int, c_int, P, P, P]),
    "ta_kmeans_merge": (c_int, [P, P, c_int, c_int, c_int, c_int, P, P, POINTER(c_int), POINTER(c_int), P]),
    "ta_comm_unique_id": (c_int, [P, c_size_t]),
    "ta_comm_create": (c_int, [P, c_int, c_int, P, c_size_t, POINTER(c_void_p)]),
    "ta_comm_destroy": (c_int, [P]),
    "ta_comm_info": (c_int, [P, POINTER(c_int), POINTER(c_int)]),
    "ta_allreduce_grads": (c_int, [P, P]),
    "ta_trainer_set_comm": (c_int, [P, P]),
    "ta_trainer_create": (c_int, [P, P, P, c_int, c_int, P, POINTER(c_void_p)]),
    "ta_trainer_destroy": (c_int, [P]),
    "ta_trainer_init_random": (c_int, [P, ctypes.c_ulonglong, c_float]),
    "ta_trainer_tensor": (c_int, [P, c_char_p, POINTER(c_void_p), POINTER(c_long), POINTER(c_long), POINTER(c_long),
                                  POINTER(c_int)]),
    "ta_trainer_sync_working": (c_int, [P]),
    "ta_trainer_zero_grad": (c_int, [P]),
    "ta_trainer_forward_backward": (c_int, [P, P, P, c_int, c_int, c_long, c_int]),
    "ta_trainer_optimizer_step": (c_int, [P, c_float, c_long, P]),
    "ta_trainer_step": (c_int, [P, P, P, c_int, c_int, c_float, c_long, c_int, P]),
    "ta_trainer_write_snapshot": (c_int, [P, c_int, c_char_p, P, P]),
    "ta_trainer_write_snapshot_bank": (c_int, [P, c_char_p, P, P, POINTER(c_int)]),
    "ta_trainer_save_checkpoint": (c_int, [P, c_char_p, c_char_p, c_long, c_long, c_int]),
    "ta_trainer_set_meta": (c_int, [P, c_char_p, c_char_p]),
    "ta_base_probe": (c_int, [c_char_p, c_char_p, P, c_char_p, c_int, c_char_p, c_int, c_char_p, c_int]),
    "ta_trainer_load_base": (c_int, [P, c_char_p, c_char_p]),
    "ta_trainer_save_optimizer": (c_int, [P, c_char_p]),
    "ta_trainer_resume": (c_int, [P, c_char_p]),
    "ta_kmeans_merge_ex": (c_int, [P, P, P, c_int, c_int, c_int, c_int, c_int, ctypes.c_ulonglong, c_int, P, P, P, P,
                                   POINTER(c_int), POINTER(c_int), P]),
    "ta_centroid_merge_dir_ex": (c_int, [P, c_char_p, c_char_p, c_int, c_int, ctypes.c_ulonglong, c_int, POINTER(c_int), POINTER(c_int)]),
    "ta_dataset_load": (c_int, [P, c_char_p, POINTER(c_void_p)]),
    "ta_dataset_destroy": (c_int, [P]),
    "ta_dataset_info": (c_int, [P, POINTER(c_long), POINTER(c_long), POINTER(c_long)]),
    "ta_dataset_seek": (c_int, [P, c_long, c_long]),
    "ta_dataset_next_batch": (c_int, [P, c_int, c_int, c_int, c_int, P, P, c_int, P]),
    "ta_mask_targets_device": (c_int, [P, P, P, c_int, c_int, P]),
    "ta_trainer_step_dataset": (c_int, [P, P, c_int, c_int, c_float, c_long, P]),
    "ta_trainer_counters": (c_int, [P, POINTER(c_long), POINTER(c_long)]),
    "ta_trainer_merge_snapshots": (c_int, [P, c_int, c_char_p, POINTER(c_int)]),
    "ta_cosine_lr": (c_float, [c_float, c_long, c_long, c_long, c_float]),
    "ta_mask_targets": (None, [P, P, c_int, c_int]),
    "ta_kaiming_init_host": (None, [P, c_int, c_int, ctypes.c_uint]),
    "ta_centroid_merge_dir": (c_int, [P, c_char_p, c_char_p, c_int, POINTER(c_int), POINTER(c_int)]),
    "ta_memcpy_h2d": (c_int, [P, P, c_size_t]),
    "ta_memcpy_d2h": (c_int, [P, P, c_size_t]),
    "ta_gemm_tokens_f32_static": (c_int, [P, c_int, c_int, c_int, c_float, P, c_long, P, c_long, P, c_long, c_int, c_int,
                                          P]),
    "ta_gemm_tokens_f32": (c_int, [P, c_int, c_int, c_int, c_float, P, c_long, P, c_long, P, c_long, c_int, c_int, P]),
}


def declare(protos) -> None:
    for name, (res, args) in protos.items():
        fn = getattr(lib, name)   # AttributeError here = the .so does not export a declared symbol
        fn.restype = res
        fn.argtypes = args


declare(_PROTOS)


def exported_symbols():
    """Names this binding expects the library to export (tests compare them with include/*.h)."""
    return sorted(_PROTOS)


class Context:
    """Owns a `ta_ctx*`; `call(name, *args)` invokes an entry point whose first parameter is the
    context and raises TAError with the library's message on a non-zero return."""

    def __init__(self, device: int = 0):
        h = c_void_p()
        rc = lib.ta_ctx_create(device, ctypes.byref(h))
        if rc != TA_OK:
            raise TAError(rc, f"ta_ctx_create(device={device}) failed: an sm_100 (B200) GPU is required")
        self.h = h
        self.device = device

    def call(self, name: str, *args):
        rc = getattr(lib, name)(self.h, *args)
        if rc != TA_OK:
            raise TAError(rc, (lib.ta_last_error(self.h) or b"").decode())
        return rc

    def check_device(self) -> None:
        st = c_int(0)
        rc = lib.ta_device_status(self.h, ctypes.byref(st))
        if rc != TA_OK:
            raise TAError(rc, f"device status {st.value}: {(lib.ta_last_error(self.h) or b'').decode()}")

    @property
    def launches(self) -> int:
        return int(lib.ta_launch_count(self.h))

    def close(self) -> None:
        if self.h:
            lib.ta_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def ptr(t) -> c_void_p:
    """Device pointer of a torch tensor (or None)."""
    return c_void_p(0) if t is None else c_void_p(t.data_ptr())


def stream_ptr() -> c_void_p:
    import torch
    return c_void_p(torch.cuda.current_stream().cuda_stream)
