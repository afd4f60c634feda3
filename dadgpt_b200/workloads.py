"""Seeded synthetic inputs for the causal-attention workloads.

All tensors come from ``numpy.random.default_rng(seed)`` (PCG64) ``standard_normal`` in fp32,
C order, multiplied by the stated scale and, where the workload is bf16, rounded to nearest-even
bf16. Every consumer (CPU oracle, reference kernels, the CUDA kernels here) is fed the same
arrays, so results do not depend on who generated them. Shards of the (batch x head) axis are
cut from the same stream, so a unit's data does not depend on the number of ranks.

No dataset stands behind these: the reference (DadGPT) trains on text, but its attention path
only ever sees activations, for which i.i.d. normal values of the right shape stand in.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


def bf16_round(x: np.ndarray) -> np.ndarray:
    """fp32 -> nearest-even bf16, returned as the uint16 bit pattern."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    rounded = u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def bf16_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


@dataclass(frozen=True)
class AttnShape:
    name: str
    BH: int
    S: int
    D: int
    scale: float
    seed: int
    input_scale: float = 1.0
    dout_seed: int | None = None
    dout_scale: float = 1.0


# The configurations the benchmark and the parity tests are quoted on.
TINY = AttnShape("tiny_fp32_B4_H4_T64_D16", 16, 64, 16, 0.25, seed=0)
TINY_D32 = AttnShape("tiny_fp32_B4_H4_T64_D32", 16, 64, 32, 32 ** -0.5, seed=0)


def gpt2(T: int = 1024) -> AttnShape:
    return AttnShape(f"gpt2_124m_B16_H12_T{T}_D64", 192, T, 64, 0.125, seed=1, input_scale=0.5,
                     dout_seed=2)


LARGE = AttnShape("large_B8_H24_T8192_D128", 192, 8192, 128, 128 ** -0.5, seed=4,
                  input_scale=0.5, dout_seed=4, dout_scale=0.5)


def qkv(shape: AttnShape, units: slice | None = None):
    """q, k, v as fp32 [BH,S,D] (drawn in that order from one stream); ``units`` cuts a shard."""
    rng = np.random.default_rng(shape.seed)
    full = (shape.BH, shape.S, shape.D)
    out = []
    for _ in range(3):
        t = rng.standard_normal(full, dtype=np.float32)
        if shape.input_scale != 1.0:
            t *= np.float32(shape.input_scale)
        out.append(t if units is None else np.ascontiguousarray(t[units]))
    return out


def dout(shape: AttnShape, units: slice | None = None):
    if shape.dout_seed is None:
        raise ValueError(f"{shape.name} has no backward workload")
    rng = np.random.default_rng(shape.dout_seed)
    full = (shape.BH, shape.S, shape.D)
    if shape.dout_seed == shape.seed:  # drawn after q, k, v from the same stream
        for _ in range(3):
            rng.standard_normal(full, dtype=np.float32)
    t = rng.standard_normal(full, dtype=np.float32)
    if shape.dout_scale != 1.0:
        t *= np.float32(shape.dout_scale)
    return t if units is None else np.ascontiguousarray(t[units])


def attn_flops(BH: int, S: int, D: int):
    """Algorithmic FLOPs with the causal convention (half of dense): (fwd, bwd)."""
    return 2.0 * BH * S * S * D, 5.0 * BH * S * S * D


def attn_bytes(BH: int, S: int, D: int, elem: int = 2):
    """Algorithmic HBM bytes, read-once/write-once: (fwd, bwd)."""
    fwd = 4 * BH * S * D * elem + BH * S * 4
    bwd = 8 * BH * S * D * elem + 2 * BH * S * 4
    return fwd, bwd


@dataclass(frozen=True)
class DecodeShape:
    name: str = "gpt2_124m_decode_B64_H12_D64"
    B: int = 64
    H: int = 12
    D: int = 64
    layers: int = 12
    steps: int = 256
    max_len: int = 1280  # initial lengths in [1,1024] plus 256 appended tokens
    seed: int = 3
    scale: float = 0.125


def decode_lengths(cfg: DecodeShape) -> np.ndarray:
    """Initial per-sequence cache lengths, uniform in [1,1024]."""
    return np.random.default_rng(cfg.seed).integers(1, 1025, cfg.B).astype(np.int32)


def decode_bytes_per_layer_call(lengths_after_append: np.ndarray, H: int, D: int,
                                elem: int = 2) -> int:
    """Algorithmic bytes of one decode call: K and V rows read once, plus the per-token vectors
    (q read, new k/v read and written, out written)."""
    B = len(lengths_after_append)
    kv = int(lengths_after_append.astype(np.int64).sum()) * 2 * H * D * elem
    vec = B * H * D * elem * 6
    return kv + vec
