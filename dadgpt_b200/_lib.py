"""ctypes binding of libdadattn.so (include/dadattn.h). No fallback: a missing library is an error."""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libdadattn.so")
SHIM_PATH = os.path.join(PKG, "libdadattn_gpuops.so")

P, I, F, U64, I64, SZ = C.c_void_p, C.c_int, C.c_float, C.c_uint64, C.c_int64, C.c_size_t

# name -> (restype, argtypes); mirrors include/dadattn.h one to one.
SIGNATURES = {
    "dadattn_last_error": (C.c_char_p, []),
    "dadattn_version": (C.c_char_p, []),
    "dadattn_flash_supported": (I, [I]),
    "dadattn_flash_fwd_f32": (I, [P, P, P, P, P, I, I, I, F, P]),
    "dadattn_flash_bwd_f32": (I, [P] * 10 + [I, I, I, F, P]),
    "dadattn_flash_fwd_f32_dropout": (I, [P, P, P, P, P, I, I, I, F, F, U64, U64, I64, P]),
    "dadattn_flash_bwd_f32_dropout": (I, [P] * 10 + [I, I, I, F, F, U64, U64, I64, P]),
    "dadattn_dropout_mask": (I, [P, I64, F, U64, U64, I64, P]),
    "dadattn_dropout_mask_bits_bytes": (SZ, [I, I]),
    "dadattn_dropout_mask_bits": (I, [P, SZ, I, I, F, U64, U64, I64, P]),
    "dadattn_flash_bf16_supported": (I, [I]),
    "dadattn_flash_fwd_bf16": (I, [P, P, P, P, P, I, I, I, F, F, U64, U64, I64, P]),
    "dadattn_flash_bwd_bf16_workspace_bytes": (SZ, [I, I, I]),
    "dadattn_flash_bwd_bf16": (I, [P, P, P, P, SZ, P, P, P, P, P, P, I, I, I, F, F, U64, U64, I64, P]),
    "dadattn_flash_fwd_bf16_masked": (I, [P, P, P, P, P, I, I, I, F, F, P, P]),
    "dadattn_flash_bwd_bf16_masked": (I, [P, P, P, P, SZ, P, P, P, P, P, P, I, I, I, F, F, P, P]),
    "dadattn_flash_fwd_bf16_strided": (I, [P, P, P, P, P, I, I, I, I, F, F, U64, U64, I64, P]),
    "dadattn_flash_bwd_bf16_strided": (I, [P, P, P, P, SZ, P, P, P, P, P, P, I, I, I, I, F, F, U64, U64, I64, P]),
    "dadattn_set_bwd_deterministic": (I, [I]),
    "dadattn_set_stage_events": (I, [P, I]),
    "dadattn_flash_f32_via_bf16_workspace_bytes": (SZ, [I, I, I]),
    "dadattn_flash_fwd_f32_via_bf16": (I, [P, P, P, P, P, I, I, I, F, P, SZ, P]),
    "dadattn_flash_bwd_f32_via_bf16": (I, [P] * 9 + [I, I, I, F, P, SZ, P]),
    "dadattn_set_f32_precision": (I, [I]),
    "dadattn_get_f32_precision": (I, []),
    "dadattn_library_scratch": (I, [SZ, P]),
    "dadattn_decode_f32": (I, [P] * 6 + [I, I, I, I, F, P]),
    "dadattn_decode_workspace_bytes": (SZ, [I, I, I, I]),
    "dadattn_decode_bf16": (I, [P] * 7 + [I, I, I, I, F, P, SZ, P]),
    "dadattn_decode_f32_batched": (I, [P] * 7 + [I, I, I, I, F, P, SZ, P]),
    "dadattn_kv_cache_fill": (I, [P, P, P, P, P, I, I, I, I, I, I, I, P]),
    "dadattn_set_decode_early_start": (I, [I]),
    "dadattn_decode_bf16_noalloc": (I, [P] * 7 + [I, I, I, I, F, P]),
    "dadattn_decode_noalloc_status": (I, [P]),
    "dadattn_device_status": (I, [P]),
}

_lib = None


class DadAttnError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"dadattn error {code}: {message}")
        self.code = code


def load() -> C.CDLL:
    """Load the CUDA library. Raises if it has not been built (python -m dadgpt_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m dadgpt_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise DadAttnError(rc, load().dadattn_last_error().decode(errors="replace"))
