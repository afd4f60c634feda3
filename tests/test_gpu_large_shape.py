"""GPU parity at the large configuration (B=8, H=24 => BH=192, T=8192, D=128, bf16) and on long
head-size-64 sequences, where the CPU oracle cannot finish whole tensors in seconds:

* sampled (batch x head, query row) pairs of the forward against the CPU oracle (one query row
  of causal attention is the oracle's decode attention over the keys 0..row);
* every element against the fp32 drop-in kernels run on the same bf16-rounded inputs (the fp32
  kernels are themselves checked against the oracle at 1e-5 / 1e-4 in test_gpu_flash_f32.py);
* a size-independent property: doubling dO doubles dQ, dK, dV exactly (a power-of-two scale
  commutes with every rounding on the way) wherever the backward is order-deterministic; the
  single-pass and the two-kernel backward agree.

Tolerances as in the build spec: forward max-abs 2e-2, lse 1e-2, gradients 3e-2 relative L2.
"""
import numpy as np
import pytest
import torch

import dadgpt_b200 as dad
from dadgpt_b200 import workloads as W
from dadgpt_b200.attention import (device_status, flash_backward_bf16_workspace_bytes,
                                   set_backward_deterministic)
from tests.gpu_util import max_abs, rel_l2

pytestmark = pytest.mark.gpu


def run_bf16(q, k, v, do, scale):
    BH, S, D = q.shape
    out, lse = torch.empty_like(q), torch.empty(BH, S, device=q.device)
    dad.gpu_flash_attention_forward_bf16(out, lse, q, k, v, BH, S, D, scale)
    grads = [torch.empty_like(q) for _ in range(3)]
    ws = torch.empty(flash_backward_bf16_workspace_bytes(BH, S, D), dtype=torch.uint8,
                     device=q.device)
    dad.gpu_flash_attention_backward_bf16(*grads, ws, do, out, lse, q, k, v, BH, S, D, scale)
    assert device_status() == 0
    return out, lse, grads, ws


def run_f32_units(q, k, v, do, scale, units):
    """The fp32 kernels on a slice of the (batch x head) axis, inputs upcast from bf16."""
    f = [t[units].float().contiguous() for t in (q, k, v, do)]
    n, S, D = f[0].shape
    out, lse = torch.empty_like(f[0]), torch.empty(n, S, device=q.device)
    dad.gpu_flash_attention_forward(out, lse, f[0], f[1], f[2], n, S, D, scale)
    grads = [torch.empty_like(out) for _ in range(3)]
    dad.gpu_flash_attention_backward(*grads, torch.empty(n, S, device=q.device), f[3], out, lse,
                                     f[0], f[1], f[2], n, S, D, scale)
    assert device_status() == 0
    return out, lse, grads


def check_rows_against_oracle(oracle, out, lse, q, k, v, scale, picks):
    for u, r in picks:
        qf = q[u, r].float().cpu().numpy()
        kf = k[u, :r + 1].float().cpu().numpy()
        vf = v[u, :r + 1].float().cpu().numpy()
        want = oracle.decode(qf[None, None], kf[None, None], vf[None, None], [r + 1], scale)[0, 0]
        assert max_abs(out[u, r].float().cpu().numpy(), want) <= 2e-2, (u, r)
        s = (kf.astype(np.float64) @ qf.astype(np.float64)) * scale
        want_lse = s.max() + np.log(np.exp(s - s.max()).sum())
        assert abs(float(lse[u, r]) - want_lse) <= 1e-2, (u, r)


def test_large_shape_T8192_D128(cuda, oracle):
    shape = W.LARGE
    q, k, v = (torch.from_numpy(a).to(cuda).to(torch.bfloat16) for a in W.qkv(shape))
    do = torch.from_numpy(W.dout(shape)).to(cuda).to(torch.bfloat16)
    BH, S, D = shape.BH, shape.S, shape.D
    out, lse, grads, ws = run_bf16(q, k, v, do, shape.scale)
    for t in (out, lse, *grads):
        assert bool(torch.isfinite(t).all())

    # sampled rows against the CPU oracle: first and last row, tile edges, a few in between
    rng = np.random.default_rng(0)
    picks = [(0, 0), (0, 127), (5, 128), (191, S - 1), (77, 4095), (100, 4096)]
    picks += [(int(rng.integers(BH)), int(rng.integers(S))) for _ in range(6)]
    check_rows_against_oracle(oracle, out, lse, q, k, v, shape.scale, picks)

    # every element of a spread of units against the fp32 kernels
    for u0 in (0, 96, 188):
        units = slice(u0, u0 + 4)
        o32, l32, g32 = run_f32_units(q, k, v, do, shape.scale, units)
        assert max_abs(out[units].float().cpu().numpy(), o32.cpu().numpy()) <= 2e-2
        assert max_abs(lse[units].cpu().numpy(), l32.cpu().numpy()) <= 1e-2
        for got, want, name in zip(grads, g32, ("dq", "dk", "dv")):
            assert rel_l2(got[units].float().cpu().numpy(), want.cpu().numpy()) <= 3e-2, (u0, name)

    # doubling dO doubles the gradients bit for bit wherever nothing is summed in arrival order:
    # dK and dV of the single-pass backward, and everything in the two-kernel backward
    g2 = [torch.empty_like(q) for _ in range(3)]
    dad.gpu_flash_attention_backward_bf16(*g2, ws, do * 2, out, lse, q, k, v, BH, S, D, shape.scale)
    assert device_status() == 0
    assert torch.equal(grads[1] * 2, g2[1]) and torch.equal(grads[2] * 2, g2[2])
    assert rel_l2((grads[0] * 2).float().cpu().numpy(), g2[0].float().cpu().numpy()) <= 1e-2
    set_backward_deterministic(True)
    try:
        d1 = [torch.empty_like(q) for _ in range(3)]
        dad.gpu_flash_attention_backward_bf16(*d1, ws, do, out, lse, q, k, v, BH, S, D, shape.scale)
        dad.gpu_flash_attention_backward_bf16(*g2, ws, do * 2, out, lse, q, k, v, BH, S, D, shape.scale)
    finally:
        set_backward_deterministic(False)
    assert device_status() == 0
    for a, b, name in zip(d1, g2, ("dq", "dk", "dv")):
        assert torch.equal(a * 2, b), name
    # and the two backward paths agree
    for a, b, name in zip(grads, d1, ("dq", "dk", "dv")):
        assert rel_l2(a.float().cpu().numpy(), b.float().cpu().numpy()) <= 1e-2, name


@pytest.mark.parametrize("S", [4096, 4000])
def test_long_sequences_D64_single_pass_backward(cuda, oracle, S):
    """Head size 64 at sequence lengths where every CTA of the persistent single-pass backward
    works through many items and the (batch x head) units are scheduled in several groups."""
    BH, D, scale = 40, 64, 0.125
    g = torch.Generator(device="cpu").manual_seed(S)
    q, k, v, do = ((torch.randn(BH, S, D, generator=g) * 0.5).to(cuda).to(torch.bfloat16)
                   for _ in range(4))
    out, lse, grads, _ = run_bf16(q, k, v, do, scale)
    picks = [(0, 0), (39, S - 1), (17, 2047), (3, 2048), (21, S // 3)]
    check_rows_against_oracle(oracle, out, lse, q, k, v, scale, picks)
    for u0 in (0, 18, 36):
        units = slice(u0, u0 + 4)
        o32, l32, g32 = run_f32_units(q, k, v, do, scale, units)
        assert max_abs(out[units].float().cpu().numpy(), o32.cpu().numpy()) <= 2e-2
        assert max_abs(lse[units].cpu().numpy(), l32.cpu().numpy()) <= 1e-2
        for got, want, name in zip(grads, g32, ("dq", "dk", "dv")):
            assert rel_l2(got[units].float().cpu().numpy(), want.cpu().numpy()) <= 3e-2, (u0, name)
