"""GPU parity of the fp32 drop-in kernels (through the C ABI) against the CPU oracle, the golden
fixtures made by the reference's host ops, and the reference's own CUDA kernels on the same GPU.

Tolerances: forward max-abs 1e-5 (fp32 bar of the build spec); gradients 1e-4 relative L2, the
reference's own FusedAttentionMatchesMaterialized bar (tests/test_backward.cpp:432-480).
"""
import os

import numpy as np
import pytest
import torch

import dadgpt_b200 as dad
from dadgpt_b200 import workloads as W
from tests.gpu_util import dev_f32, max_abs, rel_l2

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def run_fwd(q, k, v, scale, dev, **kw):
    BH, S, D = q.shape
    tq, tk, tv = (dev_f32(x, dev) for x in (q, k, v))
    out = torch.full_like(tq, float("nan"))
    lse = torch.full((BH, S), float("nan"), device=dev)
    dad.gpu_flash_attention_forward(out, lse, tq, tk, tv, BH, S, D, scale, **kw)
    return out, lse, (tq, tk, tv)


def run_bwd(dout, out, lse, tensors, scale, dev, **kw):
    tq, tk, tv = tensors
    BH, S, D = tq.shape
    dq, dk, dv = (torch.full_like(tq, float("nan")) for _ in range(3))
    delta = torch.empty(BH, S, device=dev)
    dad.gpu_flash_attention_backward(dq, dk, dv, delta, dev_f32(dout, dev), out, lse, tq, tk, tv,
                                     BH, S, D, scale, **kw)
    return [t.cpu().numpy() for t in (dq, dk, dv)]


@pytest.mark.parametrize("shape", [W.TINY, W.TINY_D32], ids=lambda s: s.name)
def test_tiny_preset_against_golden(cuda, shape):
    g = np.load(os.path.join(GOLD, f"{shape.name}.npz"))
    q, k, v = W.qkv(shape)
    out, lse, ts = run_fwd(q, k, v, shape.scale, cuda)
    assert max_abs(out.cpu().numpy(), g["out"]) <= 1e-5
    dout = np.random.default_rng(int(g["dout_seed"])).standard_normal(q.shape, dtype=np.float32)
    for got, name in zip(run_bwd(dout, out, lse, ts, shape.scale, cuda), ("dq", "dk", "dv")):
        assert rel_l2(got, g[name]) <= 1e-4, name


def test_ragged_S70_with_and_without_dropout_against_golden(cuda):
    g = np.load(os.path.join(GOLD, "ragged_S70_D64.npz"))
    rng = np.random.default_rng(int(g["seed"]))
    q, k, v, dout = (rng.standard_normal((4, 70, 64), dtype=np.float32) for _ in range(4))
    scale = 64 ** -0.5
    out, lse, ts = run_fwd(q, k, v, scale, cuda)
    assert max_abs(out.cpu().numpy(), g["out"]) <= 1e-5
    for got, name in zip(run_bwd(dout, out, lse, ts, scale, cuda), ("dq", "dk", "dv")):
        assert rel_l2(got, g[name]) <= 1e-4, name
    kw = dict(rate=float(g["rate"]), seed=int(g["drop_seed"]))
    out_d, lse_d, ts = run_fwd(q, k, v, scale, cuda, **kw)
    assert max_abs(out_d.cpu().numpy(), g["out_drop"]) <= 1e-5
    assert torch.equal(lse_d, lse)  # dropout never touches the log-sum-exp
    for got, name in zip(run_bwd(dout, out_d, lse_d, ts, scale, cuda, **kw), ("dq_drop", "dk_drop", "dv_drop")):
        assert rel_l2(got, g[name]) <= 1e-4, name


@pytest.mark.parametrize("D", [16, 32, 64, 128])
@pytest.mark.parametrize("S", [1, 31, 33, 64, 70, 127, 129, 257])
def test_shapes_against_oracle(cuda, oracle, S, D):
    rng = np.random.default_rng(1000 * D + S)
    BH = 3
    q, k, v, dout = (rng.standard_normal((BH, S, D), dtype=np.float32) for _ in range(4))
    scale = D ** -0.5
    out, lse, ts = run_fwd(q, k, v, scale, cuda)
    o_ref, lse_ref = oracle.forward(q, k, v, scale)
    assert max_abs(out.cpu().numpy(), o_ref) <= 1e-5
    assert max_abs(lse.cpu().numpy(), lse_ref) <= 1e-5
    for got, want in zip(run_bwd(dout, out, lse, ts, scale, cuda), oracle.backward(dout, q, k, v, scale)):
        assert rel_l2(got, want) <= 1e-4


def test_dropout_sharded_units_match_whole(cuda, oracle):
    # unit0 makes a shard of the (batch x head) axis see the same mask as the unsharded call
    rng = np.random.default_rng(77)
    BH, S, D = 6, 96, 32
    q, k, v, dout = (rng.standard_normal((BH, S, D), dtype=np.float32) for _ in range(4))
    kw = dict(rate=0.1, seed=42)
    whole, lse, ts = run_fwd(q, k, v, 0.2, cuda, **kw)
    part, _, _ = run_fwd(q[4:], k[4:], v[4:], 0.2, cuda, unit0=4, **kw)
    assert torch.equal(whole[4:], part)
    o_ref, _ = oracle.forward(q, k, v, 0.2, **kw)
    assert max_abs(whole.cpu().numpy(), o_ref) <= 1e-5
    for got, want in zip(run_bwd(dout, whole, lse, ts, 0.2, cuda, **kw),
                         oracle.backward(dout, q, k, v, 0.2, **kw)):
        assert rel_l2(got, want) <= 1e-4


def test_rows_beyond_S_and_neighbours_untouched(cuda):
    # canaries either side of every output: the kernels never write outside [BH,S,D] / [BH,S]
    BH, S, D = 2, 70, 64
    pad = 256
    buf = torch.full((BH * S * D + 2 * pad,), 123.0, device=cuda)
    lbuf = torch.full((BH * S + 2 * pad,), 321.0, device=cuda)
    out = buf[pad:pad + BH * S * D].view(BH, S, D)
    lse = lbuf[pad:pad + BH * S].view(BH, S)
    q, k, v = (torch.randn(BH, S, D, device=cuda) for _ in range(3))
    dad.gpu_flash_attention_forward(out, lse, q, k, v, BH, S, D, 0.125)
    torch.cuda.synchronize()
    assert (buf[:pad] == 123.0).all() and (buf[-pad:] == 123.0).all()
    assert (lbuf[:pad] == 321.0).all() and (lbuf[-pad:] == 321.0).all()
    assert torch.isfinite(out).all()


def test_unaligned_tensors_take_the_scalar_path(cuda, oracle):
    # DadGPT carves tensors out of one arena with only 4-byte alignment guaranteed
    rng = np.random.default_rng(3)
    BH, S, D = 2, 40, 32
    n = BH * S * D
    q, k, v = (rng.standard_normal((BH, S, D), dtype=np.float32) for _ in range(3))
    arena = torch.zeros(4 * n + 16, device=cuda)
    views = [arena[1 + i * n: 1 + (i + 1) * n].view(BH, S, D) for i in range(4)]
    for t, x in zip(views[:3], (q, k, v)):
        t.copy_(torch.from_numpy(x))
    lse = torch.empty(BH, S, device=cuda)
    dad.gpu_flash_attention_forward(views[3], lse, views[0], views[1], views[2], BH, S, D, 0.2)
    assert max_abs(views[3].cpu().numpy(), oracle.forward(q, k, v, 0.2)[0]) <= 1e-5


def test_errors(cuda):
    t = torch.zeros(1, 8, 48, device=cuda)
    with pytest.raises(dad._lib.DadAttnError, match="unsupported d_head 48"):
        dad.gpu_flash_attention_forward(t, torch.zeros(1, 8, device=cuda), t, t, t, 1, 8, 48, 0.1)


def test_against_reference_cuda_kernels_same_gpu(cuda):
    """Forward and backward are individually interchangeable with the reference's own kernels
    (same lse convention): ours-forward feeds the reference's backward and vice versa."""
    from oracle.oracle import RefGpu
    if not RefGpu.available():
        pytest.skip("reference CUDA library not built")
    ref = RefGpu()
    BH, S, D = 6, 200, 64
    scale = 0.125
    q, k, v, dout = (torch.randn(BH, S, D, device=cuda) for _ in range(4))
    o1, l1 = torch.empty_like(q), torch.empty(BH, S, device=cuda)
    o2, l2 = torch.empty_like(q), torch.empty(BH, S, device=cuda)
    dad.gpu_flash_attention_forward(o1, l1, q, k, v, BH, S, D, scale)
    ref.check(ref.lib.refgpu_flash_forward(o2.data_ptr(), l2.data_ptr(), q.data_ptr(), k.data_ptr(),
                                           v.data_ptr(), BH, S, D, scale))
    torch.cuda.synchronize()
    assert (o1 - o2).abs().max().item() <= 1e-5 and (l1 - l2).abs().max().item() <= 1e-5
    mine = [torch.empty_like(q) for _ in range(3)]
    theirs = [torch.empty_like(q) for _ in range(3)]
    delta = torch.empty(BH, S, device=cuda)
    dad.gpu_flash_attention_backward(*mine, delta, dout, o2, l2, q, k, v, BH, S, D, scale)
    ref.check(ref.lib.refgpu_flash_backward(*(t.data_ptr() for t in theirs), delta.data_ptr(),
                                            dout.data_ptr(), o1.data_ptr(), l1.data_ptr(),
                                            q.data_ptr(), k.data_ptr(), v.data_ptr(), BH, S, D, scale))
    torch.cuda.synchronize()
    for a, b in zip(mine, theirs):
        assert rel_l2(a.cpu().numpy(), b.cpu().numpy()) <= 1e-4
