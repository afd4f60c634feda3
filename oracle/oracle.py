"""TEST INFRASTRUCTURE — ctypes/numpy door onto the CPU oracle and the compiled reference.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this module; the
library under ``dadgpt_b200`` never does.

``Oracle``      wraps oracle/liboracle.so (this repository's C restatement).
``RefHost``     wraps oracle/_ref/libdadref_host.so (the reference's own host ops, compiled from
                the reference tree by ``make -C oracle ref``); absent where that tree is absent.
``RefGpu``      wraps oracle/_ref/libdadref_gpu.so (the reference's own CUDA kernels built for
                sm_100a); takes raw device pointers.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")


def reference_dir() -> str | None:
    """Where the DadGPT source tree lies: $DADGPT_REFERENCE_DIR if set, else a directory named
    ``reference`` beside this repository. None when neither holds the reference's ``src/``."""
    env = os.environ.get("DADGPT_REFERENCE_DIR")
    cands = [env] if env else [os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "src", "tensor_ops.cpp")):
            return os.path.abspath(c)
    return None


def build_oracle() -> str:
    """Compile liboracle.so (and the reference libraries when the reference tree exists)."""
    subprocess.run(["make", "-s", "-C", HERE, "all"], check=True)
    ref = reference_dir()
    if ref:
        subprocess.run(["make", "-s", "-C", HERE, "ref", f"REF={ref}"], check=True)
    return os.path.join(HERE, "liboracle.so")


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class Oracle:
    def __init__(self, path: str | None = None):
        path = path or os.path.join(HERE, "liboracle.so")
        if not os.path.exists(path):
            build_oracle()
        L = self.lib = C.CDLL(path)
        L.oracle_attention_forward.argtypes = [
            C.c_void_p, C.c_void_p, _f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_float,
            C.c_float, C.c_uint64, C.c_uint64, C.c_int64, C.c_int]
        L.oracle_attention_forward.restype = C.c_int
        L.oracle_attention_backward.argtypes = [
            _f32p, _f32p, _f32p, C.c_void_p, C.c_void_p, _f32p, _f32p, _f32p, _f32p, C.c_int,
            C.c_int, C.c_int, C.c_float, C.c_float, C.c_uint64, C.c_uint64, C.c_int64, C.c_int]
        L.oracle_attention_backward.restype = C.c_int
        L.oracle_dropout_mask.argtypes = [_u8p, C.c_int64, C.c_float, C.c_uint64, C.c_uint64,
                                          C.c_int64]
        L.oracle_dropout_mask.restype = None
        L.oracle_philox_uniform.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64]
        L.oracle_philox_uniform.restype = C.c_float
        L.oracle_philox4x32_10.argtypes = [C.POINTER(C.c_uint32), C.c_uint64, C.c_uint64,
                                           C.c_uint64]
        L.oracle_decode_attention_batched.argtypes = [
            _f32p, _f32p, _f32p, _f32p, _i32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float,
            C.c_int]
        L.oracle_decode_attention_batched.restype = None
        for name in ("matmul", "matmul_transposed_a", "matmul_transposed_b"):
            getattr(L, "oracle_" + name).argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int,
                                                     C.c_int]
        L.oracle_softmax.argtypes = [_f32p, _f32p, C.c_int, C.c_int]
        L.oracle_softmax_backward.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int]

    # q,k,v: [BH,S,D] float32 -> (out [BH,S,D], lse [BH,S])
    def forward(self, q, k, v, scale, rate=0.0, seed=0, offset=0, unit0=0, threads=0):
        q, k, v = _f32(q), _f32(k), _f32(v)
        BH, S, D = q.shape
        out = np.empty_like(q)
        lse = np.empty((BH, S), np.float32)
        rc = self.lib.oracle_attention_forward(
            out.ctypes.data, lse.ctypes.data, q, k, v, BH, S, D, scale, rate, seed, offset,
            unit0, threads or os.cpu_count())
        assert rc == 0
        return out, lse

    def forward_timed_only(self, q, k, v, scale, threads=0):
        """Forward without keeping outputs (CPU-baseline timing)."""
        q, k, v = _f32(q), _f32(k), _f32(v)
        BH, S, D = q.shape
        rc = self.lib.oracle_attention_forward(None, None, q, k, v, BH, S, D, scale, 0.0, 0, 0,
                                               0, threads or os.cpu_count())
        assert rc == 0

    def backward(self, dout, q, k, v, scale, rate=0.0, seed=0, offset=0, unit0=0, threads=0):
        dout, q, k, v = _f32(dout), _f32(q), _f32(k), _f32(v)
        BH, S, D = q.shape
        dq, dk, dv = np.empty_like(q), np.empty_like(q), np.empty_like(q)
        rc = self.lib.oracle_attention_backward(
            dq, dk, dv, None, None, dout, q, k, v, BH, S, D, scale, rate, seed, offset, unit0,
            threads or os.cpu_count())
        assert rc == 0
        return dq, dk, dv

    def dropout_mask(self, n, rate, seed, offset=0, first=0):
        m = np.empty(n, np.uint8)
        self.lib.oracle_dropout_mask(m, n, rate, seed, offset, first)
        return m

    def philox(self, seed, subsequence, block=0):
        w = (C.c_uint32 * 4)()
        self.lib.oracle_philox4x32_10(w, seed, subsequence, block)
        return [int(x) for x in w]

    # q: [B,H,D]; caches: [B,H,max_len,D]; lens[B] = visible keys (new token included)
    def decode(self, q, k_cache, v_cache, lens, scale, threads=0):
        q, k_cache, v_cache = _f32(q), _f32(k_cache), _f32(v_cache)
        lens = np.ascontiguousarray(lens, np.int32)
        B, H, L, D = k_cache.shape
        out = np.empty((B, H, D), np.float32)
        self.lib.oracle_decode_attention_batched(out, q, k_cache, v_cache, lens, B, H, L, D,
                                                 scale, threads or os.cpu_count())
        return out


class RefHost:
    """The reference's own host ops (src/tensor_ops.cpp, src/backward.cpp) behind ref_compose.cpp."""

    PATH = os.path.join(HERE, "_ref", "libdadref_host.so")

    @classmethod
    def available(cls):
        return os.path.exists(cls.PATH)

    def __init__(self):
        L = self.lib = C.CDLL(self.PATH)
        L.ref_attention_forward.argtypes = [C.c_void_p, _f32p, _f32p, _f32p, C.c_void_p, C.c_int,
                                            C.c_int, C.c_int, C.c_float, C.c_float, C.c_int]
        L.ref_attention_backward.argtypes = [_f32p, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p,
                                             C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float,
                                             C.c_float, C.c_int]
        L.ref_decode_attention.argtypes = [_f32p, _f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int,
                                           C.c_int, C.c_float]
        for name in ("matmul", "matmul_transposed_a", "matmul_transposed_b"):
            getattr(L, "ref_" + name).argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int]
        L.ref_softmax.argtypes = [_f32p, _f32p, C.c_int, C.c_int]
        L.ref_softmax_backward.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int]

    def forward(self, q, k, v, scale, rate=0.0, mask=None, threads=0, keep=True):
        q, k, v = _f32(q), _f32(k), _f32(v)
        BH, S, D = q.shape
        out = np.empty_like(q) if keep else None
        mp = mask.ctypes.data if mask is not None else None
        self.lib.ref_attention_forward(out.ctypes.data if keep else None, q, k, v, mp, BH, S, D,
                                       scale, rate, threads or os.cpu_count())
        return out

    def backward(self, dout, q, k, v, scale, rate=0.0, mask=None, threads=0):
        dout, q, k, v = _f32(dout), _f32(q), _f32(k), _f32(v)
        BH, S, D = q.shape
        dq, dk, dv = np.empty_like(q), np.empty_like(q), np.empty_like(q)
        mp = mask.ctypes.data if mask is not None else None
        self.lib.ref_attention_backward(dq, dk, dv, dout, q, k, v, mp, BH, S, D, scale, rate,
                                        threads or os.cpu_count())
        return dq, dk, dv

    def decode(self, q, k_cache, v_cache, length, scale):
        q, k_cache, v_cache = _f32(q), _f32(k_cache), _f32(v_cache)
        H, L, D = k_cache.shape
        out = np.empty((H, D), np.float32)
        self.lib.ref_decode_attention(out, q, k_cache, v_cache, H, L, D, length, scale)
        return out


class RefGpu:
    """The reference's own CUDA code built for sm_100a; arguments are raw device pointers."""

    PATH = os.path.join(HERE, "_ref", "libdadref_gpu.so")

    @classmethod
    def available(cls):
        return os.path.exists(cls.PATH)

    def __init__(self):
        L = self.lib = C.CDLL(self.PATH)
        P, I, F = C.c_void_p, C.c_int, C.c_float
        L.refgpu_last_error.restype = C.c_char_p
        L.refgpu_flash_supported.argtypes = [I]
        L.refgpu_flash_forward.argtypes = [P, P, P, P, P, I, I, I, F]
        L.refgpu_flash_backward.argtypes = [P] * 10 + [I, I, I, F]
        L.refgpu_dropout_forward.argtypes = [P, P, P, I, F, C.c_ulonglong]
        L.refgpu_materialized_forward.argtypes = [P] * 7 + [I, I, I, F, F, C.c_ulonglong]
        L.refgpu_materialized_backward.argtypes = [P] * 12 + [I, I, I, F, F]
        L.refgpu_decode_attention.argtypes = [P] * 7 + [I, I, I, I, F]

    def check(self, rc):
        if rc != 0:
            raise RuntimeError(self.lib.refgpu_last_error().decode())
