"""GPU: the fp32-tensor entry points that run on the bf16 tensor-core kernels (operands rounded
on the fly, as the reference's GEMMs do under gpu_set_matmul_precision(BF16),
cuda/gpu_ops.cuh:43-44), against the CPU oracle evaluated on the bf16-rounded inputs.
Tolerances of the bf16 path: forward max-abs 2e-2, lse 1e-2, gradients 3e-2 relative L2."""
import numpy as np
import pytest
import torch

import dadgpt_b200 as dad
from dadgpt_b200 import _lib
from dadgpt_b200.attention import device_status, flash_f32_via_bf16_workspace_bytes
from tests.gpu_util import max_abs, rel_l2

pytestmark = pytest.mark.gpu


def rounded(x):
    return x.to(torch.bfloat16).float()


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("S", [1, 70, 129, 300])
def test_forward_backward_against_oracle(cuda, oracle, S, D):
    BH, scale = 3, D ** -0.5
    g = torch.Generator().manual_seed(100 * D + S)
    q, k, v, do = (torch.randn(BH, S, D, generator=g).to(cuda) for _ in range(4))
    ws = torch.empty(flash_f32_via_bf16_workspace_bytes(BH, S, D), dtype=torch.uint8, device=cuda)
    out = torch.full_like(q, float("nan"))
    lse = torch.full((BH, S), float("nan"), device=cuda)
    dad.gpu_flash_attention_forward_via_bf16(out, lse, q, k, v, BH, S, D, scale, ws)
    o_ref, lse_ref = oracle.forward(*(rounded(t).cpu().numpy() for t in (q, k, v)), scale)
    assert max_abs(out.cpu().numpy(), o_ref) <= 2e-2
    assert max_abs(lse.cpu().numpy(), lse_ref) <= 1e-2
    # the output is exactly representable in bf16: the backward's rounding of it changes nothing
    assert torch.equal(out, rounded(out))

    grads = [torch.full_like(q, float("nan")) for _ in range(3)]
    dad.gpu_flash_attention_backward_via_bf16(*grads, do, out, lse, q, k, v, BH, S, D, scale, ws)
    want = oracle.backward(*(rounded(t).cpu().numpy() for t in (do, q, k, v)), scale)
    for got, ref, name in zip(grads, want, ("dq", "dk", "dv")):
        if S == 1 and name != "dv":  # exactly zero in the oracle; here fp32 summation-order noise
            assert max_abs(got.cpu().numpy(), ref) <= 1e-5, name
        else:
            assert rel_l2(got.cpu().numpy(), ref) <= 3e-2, name
    assert device_status() == 0


def test_argument_checks_and_precision_switch(cuda):
    lib = _lib.load()
    t = torch.zeros(2, 8, 64, device=cuda)
    lse = torch.zeros(2, 8, device=cuda)
    small = torch.empty(256, dtype=torch.uint8, device=cuda)
    with pytest.raises(_lib.DadAttnError) as e:
        dad.gpu_flash_attention_forward_via_bf16(t, lse, t, t, t, 2, 8, 64, 0.125, small)
    assert e.value.code == -5  # workspace too small
    t32 = torch.zeros(2, 8, 32, device=cuda)
    ws = torch.empty(1 << 20, dtype=torch.uint8, device=cuda)
    with pytest.raises(_lib.DadAttnError) as e:
        dad.gpu_flash_attention_forward_via_bf16(t32, lse, t32, t32, t32, 2, 8, 32, 0.125, ws)
    assert e.value.code == -2  # head size 32 has no tensor-core kernel
    before = lib.dadattn_get_f32_precision()
    assert lib.dadattn_set_f32_precision(1) == 0 and lib.dadattn_get_f32_precision() == 1
    assert lib.dadattn_set_f32_precision(7) == -1
    assert lib.dadattn_set_f32_precision(before) == 0
