"""GPU: the allocation-free decode entry point against the workspace-taking one.

Some callers of the decode path cannot allocate device memory while they run (all HBM already
handed to their own cache pool, or no tolerance for the stall an allocation causes), so
dadattn_decode_bf16_noalloc keeps its split-K scratch in a fixed array inside the library. This
file calls it through the C ABI twice in a row (the array is shared and keeps the previous
call's contents) and compares each result with dadattn_decode_bf16 run on identical caches.
It is collected last on purpose and also passes when run alone in a fresh process.
"""
import pytest
import torch

from dadgpt_b200 import _lib

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


def test_noalloc_decode_rejects_shapes_beyond_its_array(cuda):
    lib = _lib.load()
    B, H, L, D = 4096, 12, 1280, 64  # needs ~65 MB of records, the array holds 8 MiB
    assert lib.dadattn_decode_workspace_bytes(B, H, D, L) > (8 << 20)
    x = torch.zeros(16, dtype=torch.bfloat16, device=cuda)
    n = torch.zeros(B, dtype=torch.int32, device=cuda)
    rc = lib.dadattn_decode_bf16_noalloc(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(),
                                         x.data_ptr(), x.data_ptr(), n.data_ptr(), B, H, D, L, 0.125,
                                         None)
    assert rc == -5
    msg = lib.dadattn_last_error().decode()
    assert "no-alloc" in msg and "8388608" in msg
