"""GPU: the dropout mask is bit-exact against the CPU oracle and the reference's own kernel."""
import numpy as np
import pytest
import torch

import dadgpt_b200 as dad

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,first,misalign", [(1, 0, 0), (15, 3, 1), (4096, 0, 0), (100_003, 12345, 5),
                                             (70 * 70 * 4, 0, 0)])
def test_mask_bit_exact_vs_oracle(cuda, oracle, n, first, misalign):
    buf = torch.full((n + 64,), 7, dtype=torch.uint8, device=cuda)
    mask = buf[misalign:misalign + n]
    dad.dropout_mask(mask, 0.1, 42, 0, first)
    torch.cuda.synchronize()
    assert np.array_equal(mask.cpu().numpy(), oracle.dropout_mask(n, 0.1, 42, 0, first))
    assert (buf[:misalign] == 7).all() and (buf[misalign + n:] == 7).all()


def test_mask_offset_and_big_seed(cuda, oracle):
    n = 10_000
    for seed, offset in ((0xDEADBEEFCAFEF00D, 0), (42, 1), (42, 6), (43, 2**34 + 3)):
        mask = torch.empty(n, dtype=torch.uint8, device=cuda)
        dad.dropout_mask(mask, 0.3, seed, offset, 0)
        assert np.array_equal(mask.cpu().numpy(), oracle.dropout_mask(n, 0.3, seed, offset, 0))


def test_mask_bit_exact_vs_reference_kernel(cuda, oracle):
    """gpu_dropout_init(42) + gpu_dropout_forward(ones, rate 0.1) of the reference, run on this
    GPU, against dadattn_dropout_mask and the CPU Philox: pins the mask that the reference's own
    tests never fix."""
    from oracle.oracle import RefGpu
    if not RefGpu.available():
        pytest.skip("reference CUDA library not built")
    ref = RefGpu()
    n = 192 * 64 * 64
    ones = torch.ones(n, device=cuda)
    out = torch.empty(n, device=cuda)
    ref_mask = torch.empty(n, dtype=torch.uint8, device=cuda)
    ref.check(ref.lib.refgpu_dropout_forward(out.data_ptr(), ones.data_ptr(), ref_mask.data_ptr(),
                                             n, 0.1, 42))
    mine = torch.empty(n, dtype=torch.uint8, device=cuda)
    dad.dropout_mask(mine, 0.1, 42)
    torch.cuda.synchronize()
    assert torch.equal(mine, ref_mask)
    assert np.array_equal(ref_mask[:50_000].cpu().numpy(), oracle.dropout_mask(50_000, 0.1, 42))
    # checksum of the full mask, stable across runs
    assert int(ref_mask.sum().item()) == int(mine.sum().item())
