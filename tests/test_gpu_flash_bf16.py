"""GPU parity of the bf16 tcgen05 kernels (through the C ABI) against the CPU oracle evaluated
on the bf16-rounded inputs upcast to fp32.

Tolerances (build spec): forward max-abs 2e-2, dQ/dK/dV relative L2 3e-2, lse compared at 1e-2
absolute (bf16 products feed an fp32 log-sum-exp).
"""
import numpy as np
import pytest
import torch

import dadgpt_b200 as dad
from dadgpt_b200 import workloads as W
from dadgpt_b200.attention import (device_status, flash_backward_bf16_workspace_bytes,
                                   set_backward_deterministic)
from tests.gpu_util import dev_bf16, max_abs, rel_l2

pytestmark = pytest.mark.gpu


def fwd(q, k, v, scale, dev, **kw):
    (tq, fq), (tk, fk), (tv, fv) = (dev_bf16(x, dev) for x in (q, k, v))
    BH, S, D = q.shape
    out = torch.full_like(tq, float("nan"))
    lse = torch.full((BH, S), float("nan"), device=dev)
    dad.gpu_flash_attention_forward_bf16(out, lse, tq, tk, tv, BH, S, D, scale, **kw)
    assert device_status() == 0
    return out, lse, (tq, tk, tv), (fq, fk, fv)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("S", [1, 31, 128, 129, 200, 256, 384, 600, 700, 1100])
def test_forward_shapes_against_oracle(cuda, oracle, S, D):
    # (S = 600 and 1100: an odd number of 128-row tiles, so the last query-tile pair of the
    # head-size-64 kernel has no second tile and walks more K/V tiles than its ring holds)
    rng = np.random.default_rng(17 * D + S)
    BH = 3
    q, k, v = (rng.standard_normal((BH, S, D), dtype=np.float32) for _ in range(3))
    scale = D ** -0.5
    out, lse, _, (fq, fk, fv) = fwd(q, k, v, scale, cuda)
    o_ref, lse_ref = oracle.forward(fq, fk, fv, scale)
    assert max_abs(out.float().cpu().numpy(), o_ref) <= 2e-2
    assert max_abs(lse.cpu().numpy(), lse_ref) <= 1e-2


def test_forward_large_scores_trigger_the_lazy_rescale(cuda, oracle):
    # Row maxima that grow by much more than 2^8 from tile to tile force the O rescale path.
    rng = np.random.default_rng(5)
    BH, S, D = 2, 512, 64
    q, k, v = (rng.standard_normal((BH, S, D), dtype=np.float32) for _ in range(3))
    k *= np.linspace(0.2, 6.0, S, dtype=np.float32)[None, :, None]
    out, lse, _, (fq, fk, fv) = fwd(q, k, v, 1.0, cuda)
    o_ref, lse_ref = oracle.forward(fq, fk, fv, 1.0)
    assert max_abs(out.float().cpu().numpy(), o_ref) <= 2e-2
    assert max_abs(lse.cpu().numpy(), lse_ref) <= 2e-2


def test_forward_gpt2_shape_subset_and_properties(cuda, oracle):
    """Full GPT-2-124M shape (B=16,H=12,T=1024,D=64): a few (b,h) units against the oracle, all
    units through size-independent properties (finite; rows of a causal softmax average V, so
    |out| <= max|V| per unit; row 0 returns v[0]; deterministic across two calls)."""
    shape = W.gpt2(1024)
    q, k, v = W.qkv(shape)
    out, lse, (tq, tk, tv), (fq, fk, fv) = fwd(q, k, v, shape.scale, cuda)
    units = [0, 77, 191]
    o_ref, lse_ref = oracle.forward(fq[units], fk[units], fv[units], shape.scale)
    assert max_abs(out[units].float().cpu().numpy(), o_ref) <= 2e-2
    assert max_abs(lse[units].cpu().numpy(), lse_ref) <= 1e-2
    o = out.float()
    assert torch.isfinite(o).all() and torch.isfinite(lse).all()
    assert (o.abs().amax(dim=(1, 2)) <= tv.float().abs().amax(dim=(1, 2)) + 1e-2).all()
    assert torch.equal(out[:, 0], tv[:, 0])
    out2, lse2 = torch.empty_like(out), torch.empty_like(lse)
    dad.gpu_flash_attention_forward_bf16(out2, lse2, tq, tk, tv, shape.BH, shape.S, shape.D, shape.scale)
    assert torch.equal(out, out2) and torch.equal(lse, lse2)


@pytest.mark.parametrize("D", [64, 128])
def test_forward_dropout_against_oracle(cuda, oracle, D):
    rng = np.random.default_rng(23)
    BH, S = 3, 200
    q, k, v = (rng.standard_normal((BH, S, D), dtype=np.float32) for _ in range(3))
    scale = D ** -0.5
    kw = dict(rate=0.1, seed=42, offset=0)
    out, lse, _, (fq, fk, fv) = fwd(q, k, v, scale, cuda, **kw)
    o_ref, lse_ref = oracle.forward(fq, fk, fv, scale, **kw)
    assert max_abs(out.float().cpu().numpy(), o_ref) <= 2e-2
    assert max_abs(lse.cpu().numpy(), lse_ref) <= 1e-2
    part, _, _, _ = fwd(q[1:], k[1:], v[1:], scale, cuda, unit0=1, **kw)
    assert torch.equal(part, out[1:])


def test_bf16_matches_fp32_kernel_on_same_inputs(cuda):
    BH, S, D = 4, 300, 64
    q, k, v = (torch.randn(BH, S, D, device=cuda).to(torch.bfloat16) for _ in range(3))
    out, lse = torch.empty_like(q), torch.empty(BH, S, device=cuda)
    dad.gpu_flash_attention_forward_bf16(out, lse, q, k, v, BH, S, D, 0.125)
    o32, l32 = torch.empty(BH, S, D, device=cuda), torch.empty(BH, S, device=cuda)
    dad.gpu_flash_attention_forward(o32, l32, q.float(), k.float(), v.float(), BH, S, D, 0.125)
    assert (out.float() - o32).abs().max().item() <= 2e-2
    assert (lse - l32).abs().max().item() <= 1e-2


def bwd(dout, out, lse, tensors, scale, dev, **kw):
    tq, tk, tv = tensors
    BH, S, D = tq.shape
    tdo, fdo = dev_bf16(dout, dev)
    dq, dk, dv = (torch.full_like(tq, float("nan")) for _ in range(3))
    ws = torch.empty(flash_backward_bf16_workspace_bytes(BH, S, D), dtype=torch.uint8, device=dev)
    dad.gpu_flash_attention_backward_bf16(dq, dk, dv, ws, tdo, out, lse, tq, tk, tv, BH, S, D,
                                          scale, **kw)
    assert device_status() == 0
    return [t.float().cpu().numpy() for t in (dq, dk, dv)], fdo


@pytest.fixture(params=[False, True], ids=["single_pass", "deterministic"])
def bwd_mode(request):
    """Both backward paths: the single-pass kernels (default) and the two-kernel one."""
    set_backward_deterministic(request.param)
    yield request.param
    set_backward_deterministic(False)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("S", [1, 31, 128, 129, 200, 384, 700])
def test_backward_shapes_against_oracle(cuda, oracle, bwd_mode, S, D):
    rng = np.random.default_rng(31 * D + S)
    BH = 3
    q, k, v, dout = (rng.standard_normal((BH, S, D), dtype=np.float32) for _ in range(4))
    scale = D ** -0.5
    out, lse, ts, (fq, fk, fv) = fwd(q, k, v, scale, cuda)
    grads, fdo = bwd(dout, out, lse, ts, scale, cuda)
    for got, want, name in zip(grads, oracle.backward(fdo, fq, fk, fv, scale), ("dq", "dk", "dv")):
        assert np.isfinite(got).all(), name
        assert rel_l2(got, want) <= 3e-2, name


@pytest.mark.parametrize("shift", [1, 2, 3])
def test_backward_takes_lse_at_any_four_byte_alignment(cuda, shift):
    """The single-pass backward (head size 64) brings lse in with TMA boxes that start on 16-byte
    boundaries; an lse pointer that is only 4-byte aligned (a slice of a larger buffer) and rows
    whose offsets are odd (S = 129) must give the same gradients as the aligned call."""
    rng = np.random.default_rng(1290 + shift)
    BH, S, D = 3, 129, 64
    q, k, v, dout = (rng.standard_normal((BH, S, D), dtype=np.float32) for _ in range(4))
    scale = D ** -0.5
    out, lse, ts, _ = fwd(q, k, v, scale, cuda)
    want, _ = bwd(dout, out, lse, ts, scale, cuda)
    pool = torch.zeros(BH * S + 8, dtype=torch.float32, device=cuda)
    moved = pool[shift:shift + BH * S].view(BH, S)
    moved.copy_(lse)
    assert moved.data_ptr() % 16 == 4 * shift
    got, _ = bwd(dout, out, moved, ts, scale, cuda)
    for a, b, name in zip(got, want, ("dq", "dk", "dv")):
        if name == "dq":   # summed in arrival order: last bits may differ
            assert rel_l2(a, b) <= 1e-2
        else:
            assert np.array_equal(a, b), name


@pytest.mark.parametrize("D", [64, 128])
def test_backward_dropout_against_oracle(cuda, oracle, bwd_mode, D):
    rng = np.random.default_rng(41)
    BH, S = 3, 200
    q, k, v, dout = (rng.standard_normal((BH, S, D), dtype=np.float32) for _ in range(4))
    scale = D ** -0.5
    kw = dict(rate=0.1, seed=42, offset=0)
    out, lse, ts, (fq, fk, fv) = fwd(q, k, v, scale, cuda, **kw)
    grads, fdo = bwd(dout, out, lse, ts, scale, cuda, **kw)
    for got, want, name in zip(grads, oracle.backward(fdo, fq, fk, fv, scale, **kw), ("dq", "dk", "dv")):
        assert rel_l2(got, want) <= 3e-2, name
    # a shard of the (batch x head) axis reproduces its slice of the whole
    part, _ = bwd(dout[1:], out[1:].contiguous(), lse[1:].contiguous(), [t[1:].contiguous() for t in ts],
                  scale, cuda, unit0=1, **kw)
    for a, b, name in zip(part, grads, ("dq", "dk", "dv")):
        if name == "dq" and not bwd_mode:  # summed in arrival order: last bits may differ
            assert rel_l2(a, b[1:]) <= 1e-2
        else:
            assert np.array_equal(a, b[1:])


def test_backward_gpt2_shape_subset_and_properties(cuda, oracle, bwd_mode):
    """Full GPT-2-124M shape with dropout 0.1 (Philox seed 42, offset 0): three (b,h) units against
    the oracle (each with its own global unit index, which fixes its mask); all units: finite and
    bit-identical across two calls (dQ of the single-pass kernel: equal up to summation order)."""
    shape = W.gpt2(1024)
    q, k, v = W.qkv(shape)
    dout = W.dout(shape)
    kw = dict(rate=0.1, seed=42, offset=0)
    out, lse, ts, (fq, fk, fv) = fwd(q, k, v, shape.scale, cuda, **kw)
    grads, fdo = bwd(dout, out, lse, ts, shape.scale, cuda, **kw)
    units = [0, 100, 191]
    for u in units:
        w = oracle.backward(fdo[u:u + 1], fq[u:u + 1], fk[u:u + 1], fv[u:u + 1], shape.scale,
                            rate=0.1, seed=42, unit0=u)
        for got, ref, name in zip(grads, w, ("dq", "dk", "dv")):
            assert rel_l2(got[u:u + 1], ref) <= 3e-2, (u, name)
    for g in grads:
        assert np.isfinite(g).all()
    grads2, _ = bwd(dout, out, lse, ts, shape.scale, cuda, **kw)
    for a, b, name in zip(grads, grads2, ("dq", "dk", "dv")):
        if name == "dq" and not bwd_mode:  # the single-pass kernel sums dQ in arrival order
            assert rel_l2(a, b) <= 1e-2
        else:
            assert np.array_equal(a, b), name


def test_backward_matches_fp32_kernel_on_same_inputs(cuda):
    BH, S, D = 4, 300, 64
    q, k, v, do = (torch.randn(BH, S, D, device=cuda).to(torch.bfloat16) for _ in range(4))
    out, lse = torch.empty_like(q), torch.empty(BH, S, device=cuda)
    dad.gpu_flash_attention_forward_bf16(out, lse, q, k, v, BH, S, D, 0.125)
    dq, dk, dv = (torch.empty_like(q) for _ in range(3))
    ws = torch.empty(flash_backward_bf16_workspace_bytes(BH, S, D), dtype=torch.uint8, device=cuda)
    dad.gpu_flash_attention_backward_bf16(dq, dk, dv, ws, do, out, lse, q, k, v, BH, S, D, 0.125)
    o32, l32 = torch.empty(BH, S, D, device=cuda), torch.empty(BH, S, device=cuda)
    f = [t.float() for t in (q, k, v, do)]
    dad.gpu_flash_attention_forward(o32, l32, f[0], f[1], f[2], BH, S, D, 0.125)
    g32 = [torch.empty_like(o32) for _ in range(3)]
    dad.gpu_flash_attention_backward(*g32, torch.empty(BH, S, device=cuda), f[3], o32, l32, f[0], f[1],
                                     f[2], BH, S, D, 0.125)
    for a, b in zip((dq, dk, dv), g32):
        assert rel_l2(a.float().cpu().numpy(), b.cpu().numpy()) <= 3e-2


@pytest.mark.parametrize("BH,S,unit0", [(3, 200, 0), (2, 700, 4), (5, 1024, 187)])
def test_bit_packed_dropout_mask_gives_the_same_results_as_drawing_in_the_kernels(cuda, BH, S, unit0):
    """Forward and single-pass backward at head size 64 fed with dadattn_dropout_mask_bits
    against the same calls drawing the Philox mask themselves: out, lse, dK and dV bit for bit
    (dQ is summed in arrival order in both, so it is compared at 1e-2 relative L2)."""
    D, scale, rate = 64, 0.125, 0.1
    g = torch.Generator(device="cpu").manual_seed(BH * S)
    tq, tk, tv, tdo = ((torch.randn(BH, S, D, generator=g) * 0.7).to(cuda).to(torch.bfloat16) for _ in range(4))
    bits = dad.dropout_mask_bits(BH, S, rate, 42, 0, unit0)
    ws = torch.empty(flash_backward_bf16_workspace_bytes(BH, S, D), dtype=torch.uint8, device=cuda)
    res = []
    for kw in (dict(rate=rate, seed=42, offset=0, unit0=unit0), dict(rate=rate, mask_bits=bits)):
        out, lse = torch.full_like(tq, float("nan")), torch.full((BH, S), float("nan"), device=cuda)
        dad.gpu_flash_attention_forward_bf16(out, lse, tq, tk, tv, BH, S, D, scale, **kw)
        grads = [torch.full_like(tq, float("nan")) for _ in range(3)]
        dad.gpu_flash_attention_backward_bf16(*grads, ws, tdo, out, lse, tq, tk, tv, BH, S, D, scale, **kw)
        assert device_status() == 0
        res.append([out, lse] + grads)
    for name, a, b in zip(("out", "lse", "dq", "dk", "dv"), *res):
        assert torch.isfinite(a.float()).all(), name
        if name == "dq":
            assert rel_l2(a.float().cpu().numpy(), b.float().cpu().numpy()) <= 1e-2
        else:
            assert torch.equal(a, b), name
    # the mask actually drops something: the dropout-free forward differs
    plain, lse0 = torch.empty_like(tq), torch.empty(BH, S, device=cuda)
    dad.gpu_flash_attention_forward_bf16(plain, lse0, tq, tk, tv, BH, S, D, scale)
    assert not torch.equal(plain, res[1][0]) and torch.equal(lse0, res[1][1])


def test_masked_calls_reject_what_they_do_not_cover(cuda):
    from dadgpt_b200 import _lib
    BH, S = 1, 128
    bits = dad.dropout_mask_bits(BH, S, 0.1, 42)
    x = torch.zeros(BH, S, 128, dtype=torch.bfloat16, device=cuda)
    lse = torch.zeros(BH, S, device=cuda)
    with pytest.raises(_lib.DadAttnError, match="head size 64"):
        dad.gpu_flash_attention_forward_bf16(x, lse, x, x, x, BH, S, 128, 0.1, rate=0.1, mask_bits=bits)
    small = torch.zeros(4, dtype=torch.int32, device=cuda)
    with pytest.raises(_lib.DadAttnError, match="bytes"):
        dad.dropout_mask_bits(BH, S, 0.1, 42, out=small)


def test_forward_many_single_tile_units(cuda, oracle):
    """S = 128 with many (batch x head) units: every work item of the head-size-64 forward is a
    lone query tile, every persistent CTA walks several items, and the second softmax group and
    its issuer idle throughout (they must neither stall nor release buffers early)."""
    BH, S, D, scale = 700, 128, 64, 0.125
    g = torch.Generator(device="cpu").manual_seed(9)
    tq, tk, tv = ((torch.randn(BH, S, D, generator=g) * 0.7).to(cuda).to(torch.bfloat16) for _ in range(3))
    out, lse = torch.full_like(tq, float("nan")), torch.full((BH, S), float("nan"), device=cuda)
    dad.gpu_flash_attention_forward_bf16(out, lse, tq, tk, tv, BH, S, D, scale)
    assert device_status() == 0
    units = [0, 147, 148, 295, 296, 699]
    o_ref, lse_ref = oracle.forward(tq[units].float().cpu().numpy(), tk[units].float().cpu().numpy(),
                                    tv[units].float().cpu().numpy(), scale)
    assert max_abs(out[units].float().cpu().numpy(), o_ref) <= 2e-2
    assert max_abs(lse[units].cpu().numpy(), lse_ref) <= 1e-2
    o32, l32 = torch.empty(BH, S, D, device=cuda), torch.empty(BH, S, device=cuda)
    dad.gpu_flash_attention_forward(o32, l32, tq.float(), tk.float(), tv.float(), BH, S, D, scale)
    assert (out.float() - o32).abs().max().item() <= 2e-2 and (lse - l32).abs().max().item() <= 1e-2


@pytest.mark.parametrize("BH,S", [(1700, 128), (330, 640), (90, 1100)])
def test_forward_work_item_deals_cover_every_item_once(cuda, BH, S):
    """The head-size-64 forward hands its work items out before the launch: a greedy deal passed
    as a kernel parameter for small launches (the last two shapes), a closed-form deal for large
    ones (the first has more items than the table holds). Outputs start as NaN, so an item that
    no CTA took shows; every unit is compared with the fp32 kernel."""
    D, scale = 64, 0.125
    g = torch.Generator(device="cpu").manual_seed(BH + S)
    tq, tk, tv = ((torch.randn(BH, S, D, generator=g) * 0.7).to(cuda).to(torch.bfloat16) for _ in range(3))
    out, lse = torch.full_like(tq, float("nan")), torch.full((BH, S), float("nan"), device=cuda)
    dad.gpu_flash_attention_forward_bf16(out, lse, tq, tk, tv, BH, S, D, scale)
    assert device_status() == 0
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    o32, l32 = torch.empty(BH, S, D, device=cuda), torch.empty(BH, S, device=cuda)
    dad.gpu_flash_attention_forward(o32, l32, tq.float(), tk.float(), tv.float(), BH, S, D, scale)
    assert (out.float() - o32).abs().max().item() <= 2e-2 and (lse - l32).abs().max().item() <= 1e-2

