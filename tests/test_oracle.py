"""CPU: pins the oracle (oracle/attn_oracle.c) against known answers, the committed golden
fixtures made by the reference's host ops, and — where the reference tree is present — the
reference's host ops themselves, bit for bit."""
import os

import numpy as np
import pytest

from dadgpt_b200 import workloads as W

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_reference_known_answers(oracle):
    # tests/test_tensor_ops.cpp:8-20 (MatmulBasic), :149-163 (MatmulTransposedA) of the reference
    a = np.array([1, 2, 3, 4, 5, 6], np.float32)
    b = np.array([7, 8, 9, 10, 11, 12], np.float32)
    c = np.zeros(4, np.float32)
    oracle.lib.oracle_matmul(c, a, b, 2, 3, 2)
    assert c.tolist() == [58.0, 64.0, 139.0, 154.0]
    at = np.array([1, 4, 2, 5, 3, 6], np.float32)
    oracle.lib.oracle_matmul_transposed_a(c, at, b, 2, 3, 2)
    assert c.tolist() == [58.0, 64.0, 139.0, 154.0]
    # tests/test_tensor_ops.cpp:34-58: softmax sums to one, stays finite at 1000+
    x = np.array([1000.0, 1001.0, 1002.0], np.float32)
    y = np.zeros(3, np.float32)
    oracle.lib.oracle_softmax(y, x, 1, 3)
    assert np.isfinite(y).all() and abs(float(y.sum()) - 1.0) < 1e-5
    assert y[2] > y[1] > y[0]


def test_philox_known_answers(oracle):
    # Known-answer vectors of Philox4x32-10 (Random123 distribution, kat_vectors):
    # counter/key all zero, all ones, and the digits-of-pi vector.
    assert oracle.philox(0, 0, 0) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    ones = 0xFFFFFFFFFFFFFFFF
    assert oracle.philox(ones, ones, ones) == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    assert oracle.philox(0x299F31D0A4093822, 0x0370734413198A2E, 0x85A308D3243F6A88) == [
        0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]


def test_dropout_mask_statistics_and_determinism(oracle):
    m1 = oracle.dropout_mask(200_000, 0.1, 42)
    m2 = oracle.dropout_mask(200_000, 0.1, 42)
    assert (m1 == m2).all()
    assert abs(1.0 - m1.mean() - 0.1) < 0.005
    # a shard starting at element 1000 sees the same bits as the full mask
    assert (oracle.dropout_mask(5000, 0.1, 42, first=1000) == m1[1000:6000]).all()
    assert (oracle.dropout_mask(1000, 0.1, 43) != m1[:1000]).any()
    assert oracle.dropout_mask(100, 0.0, 1).all()


@pytest.mark.parametrize("shape", [W.TINY, W.TINY_D32], ids=lambda s: s.name)
def test_oracle_matches_golden_tiny(oracle, shape):
    g = np.load(os.path.join(GOLD, f"{shape.name}.npz"))
    q, k, v = W.qkv(shape)
    out, lse = oracle.forward(q, k, v, shape.scale)
    assert np.array_equal(out, g["out"])
    dout = np.random.default_rng(int(g["dout_seed"])).standard_normal(q.shape, dtype=np.float32)
    dq, dk, dv = oracle.backward(dout, q, k, v, shape.scale)
    assert np.array_equal(dq, g["dq"]) and np.array_equal(dk, g["dk"]) and np.array_equal(dv, g["dv"])
    # lse is the log-sum-exp of the scaled, causally masked scores (fp64 cross-check)
    s = np.einsum("bid,bjd->bij", q.astype(np.float64), k.astype(np.float64)) * shape.scale
    s = np.where(np.tril(np.ones((shape.S, shape.S), bool)), s, -np.inf)
    ref_lse = np.log(np.exp(s - s.max(-1, keepdims=True)).sum(-1)) + s.max(-1)
    assert np.abs(lse - ref_lse).max() < 1e-5


def test_oracle_matches_golden_ragged_and_dropout(oracle):
    g = np.load(os.path.join(GOLD, "ragged_S70_D64.npz"))
    rng = np.random.default_rng(int(g["seed"]))
    q, k, v, dout = (rng.standard_normal((4, 70, 64), dtype=np.float32) for _ in range(4))
    scale = 64 ** -0.5
    out, _ = oracle.forward(q, k, v, scale)
    assert np.array_equal(out, g["out"])
    for a, b in zip(oracle.backward(dout, q, k, v, scale), (g["dq"], g["dk"], g["dv"])):
        assert np.array_equal(a, b)
    rate, seed = float(g["rate"]), int(g["drop_seed"])
    out_d, lse_d = oracle.forward(q, k, v, scale, rate=rate, seed=seed)
    assert np.array_equal(out_d, g["out_drop"])
    for a, b in zip(oracle.backward(dout, q, k, v, scale, rate=rate, seed=seed),
                    (g["dq_drop"], g["dk_drop"], g["dv_drop"])):
        assert np.array_equal(a, b)
    # dropout leaves lse untouched
    assert np.array_equal(lse_d, oracle.forward(q, k, v, scale)[1])


def test_oracle_decode_matches_golden(oracle):
    g = np.load(os.path.join(GOLD, "decode_H4_L48_D32.npz"))
    rng = np.random.default_rng(int(g["seed"]))
    kc, vc = (rng.standard_normal((4, 48, 32), dtype=np.float32) for _ in range(2))
    qs = rng.standard_normal((3, 4, 32), dtype=np.float32)
    lens = g["lens"]
    out = oracle.decode(qs, np.broadcast_to(kc, (3, 4, 48, 32)).copy(),
                        np.broadcast_to(vc, (3, 4, 48, 32)).copy(), lens, 32 ** -0.5)
    assert np.array_equal(out, g["out"])


def test_decode_equals_last_row_of_full_attention(oracle):
    # The relation the reference's KVCacheMatchesFullForward test pins (tests/test_model.cpp:216-252)
    rng = np.random.default_rng(5)
    H, S, D = 3, 33, 16
    q, k, v = (rng.standard_normal((H, S, D), dtype=np.float32) for _ in range(3))
    full, _ = oracle.forward(q, k, v, 0.25)
    for pos in (0, 1, 31, 32):
        dec = oracle.decode(q[None, :, pos], k[None], v[None], np.array([pos + 1]), 0.25)[0]
        assert np.abs(dec - full[:, pos]).max() < 1e-5


def test_causality(oracle):
    # tests/test_model.cpp:97-128 of the reference: later tokens do not change earlier outputs
    rng = np.random.default_rng(9)
    q, k, v = (rng.standard_normal((2, 20, 16), dtype=np.float32) for _ in range(3))
    a, _ = oracle.forward(q, k, v, 0.25)
    k2, v2 = k.copy(), v.copy()
    k2[:, 10:] += 1.0
    v2[:, 10:] -= 2.0
    b, _ = oracle.forward(q, k2, v2, 0.25)
    assert np.array_equal(a[:, :10], b[:, :10]) and not np.array_equal(a[:, 10:], b[:, 10:])


def test_oracle_bit_equal_to_reference_host_ops(oracle, ref_host):
    rng = np.random.default_rng(21)
    for (BH, S, D) in ((3, 1, 16), (2, 31, 32), (2, 65, 64), (1, 129, 128)):
        q, k, v, dout = (rng.standard_normal((BH, S, D), dtype=np.float32) for _ in range(4))
        scale = D ** -0.5
        assert np.array_equal(oracle.forward(q, k, v, scale)[0], ref_host.forward(q, k, v, scale))
        for a, b in zip(oracle.backward(dout, q, k, v, scale), ref_host.backward(dout, q, k, v, scale)):
            assert np.array_equal(a, b)
        mask = oracle.dropout_mask(BH * S * S, 0.1, 42).reshape(BH, S, S)
        assert np.array_equal(oracle.forward(q, k, v, scale, rate=0.1, seed=42)[0],
                              ref_host.forward(q, k, v, scale, rate=0.1, mask=mask))
        for a, b in zip(oracle.backward(dout, q, k, v, scale, rate=0.1, seed=42),
                        ref_host.backward(dout, q, k, v, scale, rate=0.1, mask=mask)):
            assert np.array_equal(a, b)


def test_numpy_whole_unit_restatement_equals_the_c_oracle(oracle):
    """oracle/rowcheck.py (blockwise float64 numpy, used where the C loops would take minutes)
    against the C restatement, including a block edge inside the sequence."""
    from oracle.rowcheck import attention_unit
    rng = np.random.default_rng(33)
    for S, D, block in ((70, 64, 1024), (300, 32, 128), (257, 128, 64)):
        q, k, v, do = (rng.standard_normal((1, S, D), dtype=np.float32) * 0.5 for _ in range(4))
        scale = D ** -0.5
        o, lse = oracle.forward(q, k, v, scale)
        grads = oracle.backward(do, q, k, v, scale)
        got = attention_unit(q[0], k[0], v[0], do[0], scale, block=block)
        assert np.abs(got[0] - o[0]).max() < 1e-5 and np.abs(got[1] - lse[0]).max() < 1e-5
        for a, b in zip(got[2:], grads):
            assert np.linalg.norm(a - b[0]) / np.linalg.norm(b[0]) < 1e-5
        fo, fl = attention_unit(q[0], k[0], v[0], None, scale, block=block)
        assert np.array_equal(fo, got[0]) and np.array_equal(fl, got[1])
