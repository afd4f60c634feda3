"""GPU: the bf16 kernels on the activations as the reference's projections leave them,
[B*S, H*dh] (src/model.cpp:372-387), against the reference's own sequence split heads -> fused
attention -> merge heads (cuda/gpu_ops.cu:428-474 around src/model.cpp:390-394,568-574): the same
bits, without the seven 50 MB copies per layer."""
import pytest
import torch

import dadgpt_b200 as dad
from dadgpt_b200.attention import device_status, flash_backward_bf16_workspace_bytes
from tests.gpu_util import rel_l2

pytestmark = pytest.mark.gpu


def split_heads(x, B, H, S, D):   # [B*S, H*D] -> [B*H, S, D], what gpu_split_heads does
    return x.view(B, S, H, D).permute(0, 2, 1, 3).reshape(B * H, S, D).contiguous()


def merge_heads(x, B, H, S, D):   # [B*H, S, D] -> [B*S, H*D], what gpu_merge_heads does
    return x.view(B, H, S, D).permute(0, 2, 1, 3).reshape(B * S, H * D).contiguous()


@pytest.mark.parametrize("B,H,S,rate", [(2, 3, 200, 0.0), (3, 12, 384, 0.0), (2, 5, 257, 0.1), (1, 12, 1024, 0.0)])
def test_interleaved_equals_split_kernel_merge(cuda, B, H, S, rate):
    D, scale = 64, 0.125
    g = torch.Generator(device="cpu").manual_seed(B * 1000 + S)
    q, k, v, do = ((torch.randn(B * S, H * D, generator=g) * 0.7).to(cuda).to(torch.bfloat16) for _ in range(4))
    kw = dict(rate=rate, seed=42, offset=0, unit0=3)
    BH = B * H
    ws = torch.empty(flash_backward_bf16_workspace_bytes(BH, S, D), dtype=torch.uint8, device=cuda)

    # reference sequence: split, fused kernels on [BH,S,D], merge
    qh, kh, vh, doh = (split_heads(t, B, H, S, D) for t in (q, k, v, do))
    oh, lse_h = torch.empty_like(qh), torch.empty(BH, S, device=cuda)
    dad.gpu_flash_attention_forward_bf16(oh, lse_h, qh, kh, vh, BH, S, D, scale, **kw)
    gh = [torch.empty_like(qh) for _ in range(3)]
    dad.gpu_flash_attention_backward_bf16(*gh, ws, doh, oh, lse_h, qh, kh, vh, BH, S, D, scale, **kw)
    want = [merge_heads(oh, B, H, S, D), lse_h] + [merge_heads(t, B, H, S, D) for t in gh]

    # the same on the interleaved activations, outputs pre-filled to catch rows that are not written
    out = torch.full_like(q, float("nan"))
    lse = torch.full((BH, S), float("nan"), device=cuda)
    dad.gpu_flash_attention_forward_bf16_interleaved(out, lse, q, k, v, B, H, S, D, scale, **kw)
    grads = [torch.full_like(q, float("nan")) for _ in range(3)]
    dad.gpu_flash_attention_backward_bf16_interleaved(*grads, ws, do, out, lse, q, k, v, B, H, S, D, scale, **kw)
    assert device_status() == 0
    for name, a, b in zip(("out", "lse", "dq", "dk", "dv"), [out, lse] + grads, want):
        assert torch.isfinite(a.float()).all(), name
        if name == "dq":   # summed in arrival order in both
            assert rel_l2(a.float().cpu().numpy(), b.float().cpu().numpy()) <= 1e-2
        else:
            assert torch.equal(a, b), name


def test_interleaved_is_for_head_size_64(cuda):
    from dadgpt_b200 import _lib
    x = torch.zeros(2 * 128, 2 * 128, dtype=torch.bfloat16, device=cuda)
    lse = torch.zeros(4, 128, device=cuda)
    with pytest.raises(_lib.DadAttnError, match="head size 64"):
        dad.gpu_flash_attention_forward_bf16_interleaved(x, lse, x, x, x, 2, 2, 128, 128, 0.1)
