"""GPU: the allocation-free decode entry point against the workspace-taking one.

Some callers of the decode path cannot allocate device memory while they run (all HBM already
handed to their own cache pool, or no tolerance for the stall an allocation causes), so
dadattn_decode_bf16_noalloc keeps its split-K scratch in a fixed array inside the library. This
file calls it through the C ABI twice in a row (the array is shared and keeps the previous
call's contents) and compares each result with dadattn_decode_bf16 run on identical caches and
with the CPU oracle. It is collected last on purpose and also passes when run alone in a fresh
process.
"""
import numpy as np
import pytest
import torch

from dadgpt_b200 import _lib
from oracle.oracle import Oracle

pytestmark = pytest.mark.gpu


def _state(dev, B, H, L, D, lens, seed):
    g = torch.Generator(device=dev).manual_seed(seed)
    k = torch.randn(B, H, L, D, device=dev, generator=g).to(torch.bfloat16)
    v = torch.randn(B, H, L, D, device=dev, generator=g).to(torch.bfloat16)
    return k, v, torch.tensor(lens, dtype=torch.int32, device=dev)


def test_noalloc_decode_matches_workspace_decode_twice_in_a_row(cuda):
    lib = _lib.load()
    B, H, L, D, scale = 5, 12, 640, 64, 0.125
    lens = [0, 127, 128, 300, 637]
    stream = torch.cuda.current_stream().cuda_stream
    k1, v1, n1 = _state(cuda, B, H, L, D, lens, 1)
    k2, v2, n2 = k1.clone(), v1.clone(), n1.clone()
    ws_bytes = lib.dadattn_decode_workspace_bytes(B, H, D, L)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=cuda)
    g = torch.Generator(device=cuda).manual_seed(7)
    for call in range(2):  # the second call finds the first call's partials in the array
        q, kn, vn = (torch.randn(B, H, D, device=cuda, generator=g).to(torch.bfloat16) for _ in range(3))
        want, got = torch.zeros_like(q), torch.zeros_like(q)
        rc = lib.dadattn_decode_bf16(want.data_ptr(), q.data_ptr(), kn.data_ptr(), vn.data_ptr(),
                                     k1.data_ptr(), v1.data_ptr(), n1.data_ptr(), B, H, D, L, scale,
                                     ws.data_ptr(), ws_bytes, stream)
        assert rc == 0, lib.dadattn_last_error()
        rc = lib.dadattn_decode_bf16_noalloc(got.data_ptr(), q.data_ptr(), kn.data_ptr(),
                                             vn.data_ptr(), k2.data_ptr(), v2.data_ptr(),
                                             n2.data_ptr(), B, H, D, L, scale, stream)
        assert rc == 0, lib.dadattn_last_error()
        torch.cuda.synchronize()
        # same kernels, same inputs: the decode tests' tolerance (2e-2) is met with room to spare
        assert (got.float() - want.float()).abs().max().item() <= 2e-2
        assert torch.isfinite(got.float()).all()
        assert torch.equal(n1, n2) and n2.tolist() == [x + call + 1 for x in lens]
        assert torch.equal(k1, k2) and torch.equal(v1, v2)  # both appended the same rows
        # and against the CPU oracle on the caches as they are after the append
        ref = Oracle().decode(q.float().cpu().numpy(), k2.float().cpu().numpy(),
                              v2.float().cpu().numpy(), n2.cpu().numpy(), scale)
        assert np.abs(got.float().cpu().numpy() - ref).max() <= 2e-2
    assert lib.dadattn_decode_noalloc_status(stream) == 0


def test_noalloc_decode_reports_a_full_sequence(cuda):
    """A sequence already at max_len is left alone and noted in the entry point's own status word,
    which dadattn_decode_noalloc_status returns once and then clears."""
    lib = _lib.load()
    B, H, L, D, scale = 3, 4, 256, 64, 0.125
    stream = torch.cuda.current_stream().cuda_stream
    k, v, n = _state(cuda, B, H, L, D, [5, L, 200], 3)
    k0 = k.clone()
    g = torch.Generator(device=cuda).manual_seed(11)
    q, kn, vn = (torch.randn(B, H, D, device=cuda, generator=g).to(torch.bfloat16) for _ in range(3))
    got = torch.zeros_like(q)
    assert lib.dadattn_decode_noalloc_status(stream) == 0
    rc = lib.dadattn_decode_bf16_noalloc(got.data_ptr(), q.data_ptr(), kn.data_ptr(), vn.data_ptr(),
                                         k.data_ptr(), v.data_ptr(), n.data_ptr(), B, H, D, L, scale,
                                         stream)
    assert rc == 0, lib.dadattn_last_error()
    assert lib.dadattn_decode_noalloc_status(stream) == -1
    assert b"skipped" in lib.dadattn_last_error()
    assert lib.dadattn_decode_noalloc_status(stream) == 0  # cleared by the read
    assert n.tolist() == [6, L, 201]
    assert torch.equal(k[1], k0[1])  # the full sequence's cache is untouched
    ref = Oracle().decode(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(),
                          n.cpu().numpy(), scale)
    for b in (0, 2):
        assert np.abs(got[b].float().cpu().numpy() - ref[b]).max() <= 2e-2


def test_noalloc_decode_rejects_shapes_beyond_its_array(cuda):
    lib = _lib.load()
    B, H, L, D = 4096, 12, 1280, 64  # 49152 (sequence, head) tickets; the array has room for 16351
    x = torch.zeros(16, dtype=torch.bfloat16, device=cuda)
    n = torch.zeros(B, dtype=torch.int32, device=cuda)
    rc = lib.dadattn_decode_bf16_noalloc(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(),
                                         x.data_ptr(), x.data_ptr(), n.data_ptr(), B, H, D, L, 0.125,
                                         None)
    assert rc == -5
    msg = lib.dadattn_last_error().decode()
    assert "no-alloc" in msg and "8388608" in msg
