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


@pytest.mark.parametrize("BH,S,unit0,seed,offset,rate", [(3, 70, 0, 42, 0, 0.1), (2, 300, 5, 42, 0, 0.1),
                                                          (2, 257, 1, 7, 6, 0.1), (1, 1024, 190, 42, 0, 0.1),
                                                          (2, 200, 3, 0xDEADBEEFCAFEF00D, 8, 0.37),
                                                          (1, 130, 0, 42, 4, 0.999)])
def test_bit_packed_mask_equals_the_byte_mask(cuda, BH, S, unit0, seed, offset, rate):
    """dadattn_dropout_mask_bits against dadattn_dropout_mask (itself pinned against the
    reference's kernel above): every bit of the causal lower triangle equals the byte of the
    reference's flat [BH,S,S] mask at ((unit0 + bh) S + r) S + c; everything else is 0. Offsets
    that are multiples of 4 take the stripped-down draw with the integer drop threshold, the
    others the general one."""
    bits = dad.dropout_mask_bits(BH, S, rate, seed, offset, unit0)
    full = torch.empty(BH * S * S, dtype=torch.uint8, device=cuda)
    dad.dropout_mask(full, rate, seed, offset, unit0 * S * S)
    torch.cuda.synchronize()
    full = full.view(BH, S, S).cpu().numpy()
    nt = (S + 127) // 128
    words = bits.cpu().numpy().view(np.uint32).reshape(BH, nt * (nt + 1) // 2, 128, 4)
    unpacked = ((words[..., None] >> np.arange(32, dtype=np.uint32)) & 1).astype(np.uint8)
    unpacked = unpacked.reshape(BH, -1, 128, 128)  # [bh, tile, row, key]
    want = np.zeros_like(unpacked)
    for qt in range(nt):
        for kt in range(qt + 1):
            r0, c0 = qt * 128, kt * 128
            blk = np.zeros((BH, 128, 128), np.uint8)
            rr, cc = min(128, S - r0), min(128, S - c0)
            blk[:, :rr, :cc] = full[:, r0:r0 + rr, c0:c0 + cc]
            if qt == kt:
                blk *= np.tril(np.ones((128, 128), np.uint8))
            want[:, qt * (qt + 1) // 2 + kt] = blk
    assert np.array_equal(unpacked, want)
