"""dadgpt_b200 — B200 (sm_100a) causal attention for DadGPT behind its gpu_ops.cuh interface.

The product is the CUDA library ``libdadattn.so`` (C ABI in include/dadattn.h) plus
``libdadattn_gpuops.so``, which defines DadGPT's own ``gpu_flash_attention_*`` symbols. This
Python package is the host-side harness over that ABI: same function names and argument order as
the reference's cuda/gpu_ops.cuh, taking torch CUDA tensors for device memory and streams.
"""
from .attention import (  # noqa: F401
    KVCacheBF16,
    decode_attention_bf16,
    decode_attention_f32,
    dropout_mask,
    dropout_mask_bits,
    gpu_flash_attention_backward,
    gpu_flash_attention_backward_bf16,
    gpu_flash_attention_backward_bf16_interleaved,
    gpu_flash_attention_backward_via_bf16,
    gpu_flash_attention_forward,
    gpu_flash_attention_forward_bf16,
    gpu_flash_attention_forward_bf16_interleaved,
    gpu_flash_attention_forward_via_bf16,
    gpu_flash_attention_supported,
    set_decode_early_start,
)

__version__ = "0.1"
