"""Host-side mirror of DadGPT's fused-attention interface (reference cuda/gpu_ops.cuh:112-122).

Function names, argument order and meaning follow the reference; torch tensors stand in for its
raw device pointers, and the current torch CUDA stream for its default stream. Every function
enqueues the library's kernels and returns without synchronising, as the reference does. Errors
raise (the reference throws std::runtime_error / std::out_of_range).
"""
from __future__ import annotations

import torch

from . import _lib


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need(t: torch.Tensor, dtype, shape=None, name="tensor"):
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if t.dtype != dtype or not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous {dtype}, got {t.dtype} contiguous={t.is_contiguous()}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} has shape {tuple(t.shape)}, expected {tuple(shape)}")


def gpu_flash_attention_supported(d_head: int) -> bool:
    """reference cuda/attention.cu:232 — true for head sizes 32 and 64."""
    return d_head in (32, 64)


def gpu_flash_attention_forward(out, lse, q, k, v, BH, S, d_head, scale, *, rate=0.0, seed=0,
                                offset=0, unit0=0):
    """fp32 fused causal attention forward (reference cuda/attention.cu:234-239).

    out,q,k,v: [BH,S,d_head] fp32; lse: [BH,S] fp32. Keyword arguments add the
    attention-probability dropout of the reference's materialized branch (src/model.cpp:406-415).
    """
    lib = _lib.load()
    for n, t in (("out", out), ("q", q), ("k", k), ("v", v)):
        _need(t, torch.float32, (BH, S, d_head), n)
    _need(lse, torch.float32, (BH, S), "lse")
    _lib.check(lib.dadattn_flash_fwd_f32_dropout(_ptr(out), _ptr(lse), _ptr(q), _ptr(k), _ptr(v),
                                                 BH, S, d_head, scale, rate, seed, offset, unit0,
                                                 _stream()))


def gpu_flash_attention_backward(dq, dk, dv, delta, dout, out, lse, q, k, v, BH, S, d_head,
                                 scale, *, rate=0.0, seed=0, offset=0, unit0=0):
    """fp32 fused backward; writes dq, dk, dv (reference cuda/attention.cu:241-252)."""
    lib = _lib.load()
    for n, t in (("dq", dq), ("dk", dk), ("dv", dv), ("dout", dout), ("out", out), ("q", q),
                 ("k", k), ("v", v)):
        _need(t, torch.float32, (BH, S, d_head), n)
    _need(lse, torch.float32, (BH, S), "lse")
    _need(delta, torch.float32, None, "delta")
    if delta.numel() < BH * S:
        raise ValueError("delta scratch smaller than BH*S")
    _lib.check(lib.dadattn_flash_bwd_f32_dropout(
        _ptr(dq), _ptr(dk), _ptr(dv), _ptr(delta), _ptr(dout), _ptr(out), _ptr(lse), _ptr(q),
        _ptr(k), _ptr(v), BH, S, d_head, scale, rate, seed, offset, unit0, _stream()))


def gpu_flash_attention_forward_bf16(out, lse, q, k, v, BH, S, d_head, scale, *, rate=0.0,
                                     seed=0, offset=0, unit0=0, mask_bits=None):
    """bf16 tensor-core forward (tcgen05); same argument order as the fp32 call. With
    ``mask_bits`` (from :func:`dropout_mask_bits`) the dropout mask is read, not drawn."""
    lib = _lib.load()
    for n, t in (("out", out), ("q", q), ("k", k), ("v", v)):
        _need(t, torch.bfloat16, (BH, S, d_head), n)
    _need(lse, torch.float32, (BH, S), "lse")
    if mask_bits is not None:
        _lib.check(lib.dadattn_flash_fwd_bf16_masked(_ptr(out), _ptr(lse), _ptr(q), _ptr(k), _ptr(v),
                                                     BH, S, d_head, scale, rate, _ptr(mask_bits),
                                                     _stream()))
        return
    _lib.check(lib.dadattn_flash_fwd_bf16(_ptr(out), _ptr(lse), _ptr(q), _ptr(k), _ptr(v), BH, S,
                                          d_head, scale, rate, seed, offset, unit0, _stream()))


def dropout_mask_bits(BH, S, rate, seed, offset=0, unit0=0, out=None):
    """Bit-packed keep mask of the reference's attention dropout (cuda/gpu_ops.cu:712-734 drawn
    per probability, here packed per 128 x 128 tile of the causal lower triangle) for the
    ``mask_bits`` argument of the bf16 calls below. Returns the int32 device tensor."""
    lib = _lib.load()
    nbytes = int(lib.dadattn_dropout_mask_bits_bytes(BH, S))
    if out is None:
        out = torch.empty(nbytes // 4, dtype=torch.int32, device="cuda")
    _need(out, torch.int32, None, "mask bits")
    _lib.check(lib.dadattn_dropout_mask_bits(_ptr(out), out.numel() * 4, BH, S, rate, seed, offset,
                                             unit0, _stream()))
    return out


def flash_backward_bf16_workspace_bytes(BH, S, d_head) -> int:
    return int(_lib.load().dadattn_flash_bwd_bf16_workspace_bytes(BH, S, d_head))


def gpu_flash_attention_backward_bf16(dq, dk, dv, workspace, dout, out, lse, q, k, v, BH, S,
                                      d_head, scale, *, rate=0.0, seed=0, offset=0, unit0=0,
                                      mask_bits=None):
    """bf16 tensor-core backward; ``workspace`` replaces the fp32 call's ``delta`` scratch. With
    ``mask_bits`` (from :func:`dropout_mask_bits`) the dropout mask is read, not drawn."""
    lib = _lib.load()
    for n, t in (("dq", dq), ("dk", dk), ("dv", dv), ("dout", dout), ("out", out), ("q", q),
                 ("k", k), ("v", v)):
        _need(t, torch.bfloat16, (BH, S, d_head), n)
    _need(lse, torch.float32, (BH, S), "lse")
    nbytes = workspace.numel() * workspace.element_size()
    if mask_bits is not None:
        _lib.check(lib.dadattn_flash_bwd_bf16_masked(
            _ptr(dq), _ptr(dk), _ptr(dv), _ptr(workspace), nbytes, _ptr(dout), _ptr(out), _ptr(lse),
            _ptr(q), _ptr(k), _ptr(v), BH, S, d_head, scale, rate, _ptr(mask_bits), _stream()))
        return
    _lib.check(lib.dadattn_flash_bwd_bf16(
        _ptr(dq), _ptr(dk), _ptr(dv), _ptr(workspace), nbytes, _ptr(dout), _ptr(out), _ptr(lse),
        _ptr(q), _ptr(k), _ptr(v), BH, S, d_head, scale, rate, seed, offset, unit0, _stream()))


def gpu_flash_attention_forward_bf16_interleaved(out, lse, q, k, v, B, H, S, d_head, scale, *, rate=0.0,
                                                 seed=0, offset=0, unit0=0):
    """bf16 forward on the activations as the projections leave them, [B*S, H*d_head] (reference
    src/model.cpp:372-387): no gpu_split_heads / gpu_merge_heads copies around the call."""
    lib = _lib.load()
    for n, t in (("out", out), ("q", q), ("k", k), ("v", v)):
        _need(t, torch.bfloat16, (B * S, H * d_head), n)
    _need(lse, torch.float32, (B * H, S), "lse")
    _lib.check(lib.dadattn_flash_fwd_bf16_strided(_ptr(out), _ptr(lse), _ptr(q), _ptr(k), _ptr(v), B, H, S,
                                                  d_head, scale, rate, seed, offset, unit0, _stream()))


def gpu_flash_attention_backward_bf16_interleaved(dq, dk, dv, workspace, dout, out, lse, q, k, v, B, H, S,
                                                  d_head, scale, *, rate=0.0, seed=0, offset=0, unit0=0):
    """Backward of the call above; every bf16 tensor is [B*S, H*d_head]."""
    lib = _lib.load()
    for n, t in (("dq", dq), ("dk", dk), ("dv", dv), ("dout", dout), ("out", out), ("q", q),
                 ("k", k), ("v", v)):
        _need(t, torch.bfloat16, (B * S, H * d_head), n)
    _need(lse, torch.float32, (B * H, S), "lse")
    nbytes = workspace.numel() * workspace.element_size()
    _lib.check(lib.dadattn_flash_bwd_bf16_strided(
        _ptr(dq), _ptr(dk), _ptr(dv), _ptr(workspace), nbytes, _ptr(dout), _ptr(out), _ptr(lse),
        _ptr(q), _ptr(k), _ptr(v), B, H, S, d_head, scale, rate, seed, offset, unit0, _stream()))


def flash_f32_via_bf16_workspace_bytes(BH, S, d_head) -> int:
    return int(_lib.load().dadattn_flash_f32_via_bf16_workspace_bytes(BH, S, d_head))


def gpu_flash_attention_forward_via_bf16(out, lse, q, k, v, BH, S, d_head, scale, workspace):
    """fp32 tensors, bf16 tensor-core arithmetic: what the reference's fp32 signature
    (cuda/attention.cu:234-239) computes when its GEMM precision is BF16 (cuda/gpu_ops.cuh:43-44)."""
    lib = _lib.load()
    for n, t in (("out", out), ("q", q), ("k", k), ("v", v)):
        _need(t, torch.float32, (BH, S, d_head), n)
    _need(lse, torch.float32, (BH, S), "lse")
    nbytes = workspace.numel() * workspace.element_size()
    _lib.check(lib.dadattn_flash_fwd_f32_via_bf16(_ptr(out), _ptr(lse), _ptr(q), _ptr(k), _ptr(v),
                                                  BH, S, d_head, scale, _ptr(workspace), nbytes,
                                                  _stream()))


def gpu_flash_attention_backward_via_bf16(dq, dk, dv, dout, out, lse, q, k, v, BH, S, d_head, scale,
                                          workspace):
    """Backward of the call above (reference cuda/attention.cu:241-252; no ``delta`` argument:
    the workspace holds it)."""
    lib = _lib.load()
    for n, t in (("dq", dq), ("dk", dk), ("dv", dv), ("dout", dout), ("out", out), ("q", q),
                 ("k", k), ("v", v)):
        _need(t, torch.float32, (BH, S, d_head), n)
    _need(lse, torch.float32, (BH, S), "lse")
    nbytes = workspace.numel() * workspace.element_size()
    _lib.check(lib.dadattn_flash_bwd_f32_via_bf16(
        _ptr(dq), _ptr(dk), _ptr(dv), _ptr(dout), _ptr(out), _ptr(lse), _ptr(q), _ptr(k), _ptr(v),
        BH, S, d_head, scale, _ptr(workspace), nbytes, _stream()))


def set_backward_deterministic(on: bool) -> None:
    """Head size 64: choose between the single-pass backward (default; dQ summed across key tiles
    in arrival order, so its last bits may vary between runs) and the two-kernel backward that,
    like the reference, accumulates nothing across thread blocks."""
    _lib.check(_lib.load().dadattn_set_bwd_deterministic(1 if on else 0))


def dropout_mask(mask: torch.Tensor, rate: float, seed: int, offset: int = 0, first: int = 0):
    """Fill ``mask`` (uint8, flat) with the reference's keep(1)/drop(0) mask
    (reference cuda/gpu_ops.cu:712-734) for elements first .. first+numel-1."""
    _need(mask, torch.uint8, None, "mask")
    _lib.check(_lib.load().dadattn_dropout_mask(_ptr(mask), mask.numel(), rate, seed, offset,
                                                first, _stream()))


def decode_attention_f32(out, q, k_new, v_new, k_cache, v_cache, pos, scale):
    """Attention part of model_forward_cached (reference src/model.cpp:745-790) for one sequence:
    caches [H,max_len,D] fp32, q/k_new/v_new/out [H*D]. Raises IndexError when pos is outside
    the cache (the reference throws std::out_of_range, src/model.cpp:693-696)."""
    H, max_len, D = k_cache.shape
    if pos < 0 or pos >= max_len:
        raise IndexError(f"model_forward_cached: pos {pos} outside context length {max_len}")
    for n, t in (("out", out), ("q", q), ("k_new", k_new), ("v_new", v_new)):
        _need(t, torch.float32, None, n)
    _need(k_cache, torch.float32, (H, max_len, D), "k_cache")
    _need(v_cache, torch.float32, (H, max_len, D), "v_cache")
    _lib.check(_lib.load().dadattn_decode_f32(_ptr(out), _ptr(q), _ptr(k_new), _ptr(v_new),
                                              _ptr(k_cache), _ptr(v_cache), H, max_len, D, pos,
                                              scale, _stream()))


class KVCacheBF16:
    """Batched counterpart of the reference's ``struct KVCache`` (src/model.hpp:140-152) for one
    layer: k, v [B,H,max_len,D] bf16, per-sequence lengths on the device, split-K workspace."""

    def __init__(self, B, H, max_len, D, device="cuda"):
        self.B, self.H, self.max_len, self.D = B, H, max_len, D
        self.k = torch.zeros(B, H, max_len, D, dtype=torch.bfloat16, device=device)
        self.v = torch.zeros_like(self.k)
        self.lengths = torch.zeros(B, dtype=torch.int32, device=device)
        nbytes = int(_lib.load().dadattn_decode_workspace_bytes(B, H, D, max_len))
        # zero-filled once: the split-K tickets must start at zero (include/dadattn.h)
        self.workspace = torch.zeros(nbytes, dtype=torch.uint8, device=device)


def decode_attention_bf16(out, q, k_new, v_new, cache: KVCacheBF16, scale):
    """One decode step for every sequence of ``cache``: append k_new/v_new [B,H,D] at each
    sequence's length, attend, write out [B,H,D], lengths += 1."""
    B, H, D = cache.B, cache.H, cache.D
    for n, t in (("out", out), ("q", q), ("k_new", k_new), ("v_new", v_new)):
        _need(t, torch.bfloat16, (B, H, D), n)
    _lib.check(_lib.load().dadattn_decode_bf16(
        _ptr(out), _ptr(q), _ptr(k_new), _ptr(v_new), _ptr(cache.k), _ptr(cache.v),
        _ptr(cache.lengths), B, H, D, cache.max_len, scale, _ptr(cache.workspace),
        cache.workspace.numel(), _stream()))


def set_decode_early_start(on: bool) -> None:
    """Let :func:`decode_attention_bf16` calls of this thread fetch the lengths and their first
    cache rows while the kernel ahead of them in the stream drains. Only valid when that kernel
    does not write this call's cache, lengths or workspace (layers of a model with two or more
    layers, each with its own :class:`KVCacheBF16`); see include/dadattn.h."""
    _lib.check(_lib.load().dadattn_set_decode_early_start(1 if on else 0))


def device_status() -> int:
    """Synchronise and return (then clear) the device-side status word; 0 = no condition."""
    return int(_lib.load().dadattn_device_status(_stream()))
