"""GPU parity of the KV-cache decode kernels against the CPU oracle and the golden fixture."""
import os

import numpy as np
import pytest
import torch

import dadgpt_b200 as dad
from dadgpt_b200.attention import device_status
from tests.gpu_util import dev_f32, max_abs

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_decode_f32_against_golden(cuda):
    g = np.load(os.path.join(GOLD, "decode_H4_L48_D32.npz"))
    rng = np.random.default_rng(int(g["seed"]))
    kc, vc = (rng.standard_normal((4, 48, 32), dtype=np.float32) for _ in range(2))
    qs = rng.standard_normal((3, 4, 32), dtype=np.float32)
    for i, n in enumerate(g["lens"]):
        pos = int(n) - 1
        tk, tv = dev_f32(kc, cuda), dev_f32(vc, cuda)
        k_new, v_new = tk[:, pos].contiguous(), tv[:, pos].contiguous()
        tk[:, pos] = 0  # the call itself must append the token's k, v
        tv[:, pos] = 0
        out = torch.empty(4, 32, device=cuda)
        dad.decode_attention_f32(out, dev_f32(qs[i], cuda), k_new, v_new, tk, tv, pos, 32 ** -0.5)
        assert max_abs(out.cpu().numpy(), g["out"][i]) <= 1e-5
        assert torch.equal(tk, dev_f32(kc, cuda)) and torch.equal(tv, dev_f32(vc, cuda))


@pytest.mark.parametrize("D", [16, 64, 128])
def test_incremental_decode_equals_full_causal_forward(cuda, D):
    # the relation pinned by the reference's KVCacheMatchesFullForward (tests/test_model.cpp:216-252),
    # including the last slot of the context
    H, S = 3, 37
    q, k, v = (torch.randn(H, S, D, device=cuda) for _ in range(3))
    full, lse = torch.empty_like(q), torch.empty(H, S, device=cuda)
    scale = D ** -0.5
    dad.gpu_flash_attention_forward(full, lse, q, k, v, H, S, D, scale)
    kc, vc = torch.zeros(H, S, D, device=cuda), torch.zeros(H, S, D, device=cuda)
    for pos in range(S):
        out = torch.empty(H, D, device=cuda)
        dad.decode_attention_f32(out, q[:, pos].contiguous(), k[:, pos].contiguous(),
                                 v[:, pos].contiguous(), kc, vc, pos, scale)
        assert (out - full[:, pos]).abs().max().item() <= 1e-4  # the reference's own bar
    assert torch.equal(kc, k) and torch.equal(vc, v)


def test_decode_f32_rejects_positions_outside_the_cache(cuda):
    # reference: std::out_of_range (src/model.cpp:693-696, tests/test_model.cpp:254-277)
    kc = torch.zeros(2, 8, 16, device=cuda)
    x = torch.zeros(2, 16, device=cuda)
    for pos in (-1, 8, 100):
        with pytest.raises(IndexError):
            dad.decode_attention_f32(x, x, x, x, kc, kc.clone(), pos, 0.25)


@pytest.mark.parametrize("D", [64, 128])
def test_batched_bf16_decode_against_oracle(cuda, oracle, D):
    B, H, L = 7, 5, 700
    cache = dad.KVCacheBF16(B, H, L, D, device=cuda)
    cache.k.copy_(torch.randn(B, H, L, D, device=cuda))
    cache.v.copy_(torch.randn(B, H, L, D, device=cuda))
    lens = torch.tensor([0, 1, 127, 128, 129, 511, 699], dtype=torch.int32, device=cuda)
    cache.lengths.copy_(lens)
    scale = D ** -0.5
    for step in range(2):
        q, kn, vn = (torch.randn(B, H, D, device=cuda).to(torch.bfloat16) for _ in range(3))
        out = torch.empty_like(q)
        if step == 1:
            cache.lengths[-1] = 5  # the full sequence is replaced so that step 2 stays in range
        before = cache.lengths.clone()
        dad.decode_attention_bf16(out, q, kn, vn, cache, scale)
        torch.cuda.synchronize()
        assert torch.equal(cache.lengths, before + 1)
        for b in range(B):  # appended rows hold the new token
            assert torch.equal(cache.k[b, :, int(before[b])], kn[b])
            assert torch.equal(cache.v[b, :, int(before[b])], vn[b])
        want = oracle.decode(q.float().cpu().numpy(), cache.k.float().cpu().numpy(),
                             cache.v.float().cpu().numpy(), cache.lengths.cpu().numpy(), scale)
        assert max_abs(out.float().cpu().numpy(), want) <= 2e-2
    assert device_status() == 0


def test_many_sequences_with_tied_lengths_are_each_attended_once(cuda, oracle):
    """Enough (sequence, head) pairs that the CTAs no longer fit the GPU at once: the kernel then
    takes the sequences longest first, ranking the lengths itself. Tied and adjacent lengths are
    the hard case for that ranking (every CTA must arrive at the same order, also while other
    CTAs finish); every pair must still be attended exactly once, over several steps."""
    B, H, L, D = 48, 12, 160, 64
    cache = dad.KVCacheBF16(B, H, L, D, device=cuda)
    cache.k.copy_(torch.randn(B, H, L, D, device=cuda))
    cache.v.copy_(torch.randn(B, H, L, D, device=cuda))
    g = torch.Generator().manual_seed(11)
    lens = torch.randint(100, 104, (B,), generator=g, dtype=torch.int32)
    lens[::7] = 30
    cache.lengths.copy_(lens.to(cuda))
    scale = D ** -0.5
    for step in range(3):
        q, kn, vn = (torch.randn(B, H, D, device=cuda).to(torch.bfloat16) for _ in range(3))
        out = torch.full_like(q, float("nan"))
        before = cache.lengths.clone()
        dad.decode_attention_bf16(out, q, kn, vn, cache, scale)
        torch.cuda.synchronize()
        assert torch.equal(cache.lengths, before + 1)
        want = oracle.decode(q.float().cpu().numpy(), cache.k.float().cpu().numpy(),
                             cache.v.float().cpu().numpy(), cache.lengths.cpu().numpy(), scale)
        assert max_abs(out.float().cpu().numpy(), want) <= 2e-2
    assert device_status() == 0


def test_full_sequence_is_skipped_and_reported(cuda):
    B, H, L, D = 2, 2, 16, 64
    cache = dad.KVCacheBF16(B, H, L, D, device=cuda)
    cache.lengths.copy_(torch.tensor([3, 16], dtype=torch.int32))
    x = torch.randn(B, H, D, device=cuda).to(torch.bfloat16)
    out = torch.zeros_like(x)
    dad.decode_attention_bf16(out, x, x, x, cache, 0.125)
    assert device_status() == -1          # DADATTN_E_ARG recorded by the kernel, no fault
    assert cache.lengths.tolist() == [4, 16]
    assert (out[1] == 0).all() and device_status() == 0


def test_early_start_over_rotating_layer_caches(cuda, oracle):
    """dadattn_set_decode_early_start with the use it is meant for: several layer caches, each
    with its own lengths and workspace, decoded one after the other for several steps, so that
    the kernel ahead of a call always belongs to another cache. Every layer's output, appended
    rows and lengths are checked against the oracle at every step."""
    layers, B, H, L, D, scale = 3, 40, 12, 300, 64, 0.125
    g = torch.Generator(device=cuda).manual_seed(5)
    caches = [dad.KVCacheBF16(B, H, L, D, device=cuda) for _ in range(layers)]
    lens0 = torch.randint(1, 250, (B,), generator=torch.Generator().manual_seed(6), dtype=torch.int32)
    for c in caches:
        c.k.copy_(torch.randn(c.k.shape, device=cuda, generator=g))
        c.v.copy_(torch.randn(c.v.shape, device=cuda, generator=g))
        c.lengths.copy_(lens0.to(cuda))
    dad.set_decode_early_start(True)
    try:
        for step in range(3):
            q, kn, vn = (torch.randn(layers, B, H, D, device=cuda, generator=g).to(torch.bfloat16) for _ in range(3))
            out = torch.full_like(q, float("nan"))
            for l, c in enumerate(caches):   # back to back, no synchronisation in between
                dad.decode_attention_bf16(out[l], q[l], kn[l], vn[l], c, scale)
            torch.cuda.synchronize()
            now = (lens0 + step + 1).numpy().astype(np.int32)
            for l, c in enumerate(caches):
                assert (c.lengths.cpu().numpy() == now).all()
                want = oracle.decode(q[l].float().cpu().numpy(), c.k.float().cpu().numpy(),
                                     c.v.float().cpu().numpy(), now, scale)
                assert max_abs(out[l].float().cpu().numpy(), want) <= 2e-2
                rows = torch.from_numpy(now.astype(np.int64) - 1).to(cuda)
                ar = torch.arange(B, device=cuda)
                assert torch.equal(c.k[ar, :, rows], kn[l]) and torch.equal(c.v[ar, :, rows], vn[l])
    finally:
        dad.set_decode_early_start(False)
    assert device_status() == 0


@pytest.mark.parametrize("graph", [False, True], ids=["plain", "graph"])
def test_decode_at_the_benchmark_configuration(cuda, oracle, graph):
    """The exact decode configuration bench.py times: 64 sequences, 12 heads, head size 64,
    max_len 1280, lengths from seed 3 (every CTA walks a whole sequence, sequences taken longest
    first), several appended steps, once through plain calls and once replayed from a captured
    CUDA graph as the benchmark does. Output, appended cache rows and lengths are checked
    against the CPU oracle after every step."""
    from dadgpt_b200 import workloads as W
    cfg = W.DecodeShape()
    lens0 = W.decode_lengths(cfg)
    assert (cfg.B, cfg.H, cfg.D, cfg.max_len) == (64, 12, 64, 1280) and lens0.max() <= 1024
    cache = dad.KVCacheBF16(cfg.B, cfg.H, cfg.max_len, cfg.D, device=cuda)
    gen = torch.Generator(device=cuda).manual_seed(cfg.seed)
    cache.k.copy_(torch.randn(cache.k.shape, device=cuda, generator=gen))
    cache.v.copy_(torch.randn(cache.v.shape, device=cuda, generator=gen))
    cache.lengths.copy_(torch.from_numpy(lens0))
    q, kn, vn = (torch.empty(cfg.B, cfg.H, cfg.D, dtype=torch.bfloat16, device=cuda) for _ in range(3))
    out = torch.empty_like(q)

    def fresh_token():
        for t in (q, kn, vn):
            t.copy_(torch.randn(t.shape, device=cuda, generator=gen))

    fresh_token()
    if graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            dad.decode_attention_bf16(out, q, kn, vn, cache, cfg.scale)  # first call outside capture
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                dad.decode_attention_bf16(out, q, kn, vn, cache, cfg.scale)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        cache.lengths.copy_(torch.from_numpy(lens0))  # undo the warm-up call's advance
        step = g.replay
    else:
        def step():
            dad.decode_attention_bf16(out, q, kn, vn, cache, cfg.scale)
    for s in range(4):
        fresh_token()
        out.fill_(float("nan"))
        step()
        torch.cuda.synchronize()
        now = lens0 + s + 1
        assert (cache.lengths.cpu().numpy() == now).all()
        kc, vc = cache.k.float().cpu().numpy(), cache.v.float().cpu().numpy()
        for b in range(cfg.B):  # the appended rows hold the new token, bit for bit
            assert torch.equal(cache.k[b, :, int(now[b]) - 1], kn[b])
            assert torch.equal(cache.v[b, :, int(now[b]) - 1], vn[b])
        want = oracle.decode(q.float().cpu().numpy(), kc, vc, now.astype(np.int32), cfg.scale)
        assert max_abs(out.float().cpu().numpy(), want) <= 2e-2
    assert device_status() == 0


@pytest.mark.parametrize("D", [32, 64])
def test_batched_f32_decode_and_cache_fill(cuda, oracle, D):
    """dadattn_kv_cache_fill (a prefill's [H, n, D] heads into rows 0..n-1 of one sequence of a
    batched cache, fp32 and bf16) and dadattn_decode_f32_batched against the oracle and against
    one dadattn_decode_f32 call per sequence."""
    from dadgpt_b200 import _lib
    lib = _lib.load()
    B, H, L, scale = 5, 4, 96, D ** -0.5
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device=cuda).manual_seed(D)
    kc = torch.zeros(B, H, L, D, device=cuda)
    vc = torch.zeros_like(kc)
    kb, vb = kc.to(torch.bfloat16), vc.to(torch.bfloat16)
    lens = torch.zeros(B, dtype=torch.int32, device=cuda)
    prompts = [1, 17, 40, 63, 95]
    heads = []
    for b, n in enumerate(prompts):
        kh, vh = (torch.randn(H, n, D, device=cuda, generator=g) for _ in range(2))
        heads.append((kh, vh))
        for cache_k, cache_v, is_bf16, ln in ((kc, vc, 0, lens), (kb, vb, 1, None)):
            rc = lib.dadattn_kv_cache_fill(cache_k.data_ptr(), cache_v.data_ptr(),
                                           ln.data_ptr() if ln is not None else None, kh.data_ptr(),
                                           vh.data_ptr(), b, B, H, n, L, D, is_bf16, stream)
            assert rc == 0, lib.dadattn_last_error()
    torch.cuda.synchronize()
    assert lens.tolist() == prompts
    for b, (kh, vh) in enumerate(heads):
        n = prompts[b]
        assert torch.equal(kc[b, :, :n], kh) and torch.equal(vc[b, :, :n], vh)
        assert (kc[b, :, n:] == 0).all()
        assert torch.equal(kb[b, :, :n], kh.to(torch.bfloat16)) and torch.equal(vb[b, :, :n], vh.to(torch.bfloat16))
    # one batched decode step against the oracle and against per-sequence calls
    ws_bytes = lib.dadattn_decode_workspace_bytes(B, H, D, L)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=cuda)
    q, kn, vn = (torch.randn(B, H, D, device=cuda, generator=g) for _ in range(3))
    out = torch.full_like(q, float("nan"))
    single_k, single_v = kc.clone(), vc.clone()
    rc = lib.dadattn_decode_f32_batched(out.data_ptr(), q.data_ptr(), kn.data_ptr(), vn.data_ptr(), kc.data_ptr(),
                                        vc.data_ptr(), lens.data_ptr(), B, H, D, L, scale, ws.data_ptr(),
                                        ws_bytes, stream)
    assert rc == 0, lib.dadattn_last_error()
    torch.cuda.synchronize()
    assert lens.tolist() == [n + 1 for n in prompts]
    want = oracle.decode(q.cpu().numpy(), kc.cpu().numpy(), vc.cpu().numpy(), lens.cpu().numpy(), scale)
    assert max_abs(out.cpu().numpy(), want) <= 1e-5
    for b, n in enumerate(prompts):
        o1 = torch.empty(H, D, device=cuda)
        dad.decode_attention_f32(o1, q[b].contiguous(), kn[b].contiguous(), vn[b].contiguous(), single_k[b],
                                 single_v[b], n, scale)
        assert (o1 - out[b]).abs().max().item() <= 1e-5
        assert torch.equal(single_k[b], kc[b]) and torch.equal(single_v[b], vc[b])
    assert device_status() == 0
