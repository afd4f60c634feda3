"""TEST INFRASTRUCTURE — whole-unit causal attention in numpy, for shapes where the C oracle's
naive loops would take minutes (T = 8192, D = 128: one (batch, head) unit is ~10^11 scalar
multiply-adds there, a few seconds of BLAS here).

Same arithmetic as oracle/attn_oracle.c, i.e. as the reference's materialized attention
(src/model.cpp:396-419 forward, :576-615 backward), evaluated in float64 one block of query rows
at a time:
    forward   S = Q K^T * scale; causal mask (key c visible to row r iff c <= r,
              cuda/gpu_ops.cu:477-485); P = row softmax (src/tensor_ops.cpp:32-55); O = P V;
              lse = rowmax + ln(rowsum) of the scaled scores (cuda/attention.cu:71)
    backward  dV = P^T dO; dP = dO V^T; dS = P * (dP - rowsum(dP * P)) (src/backward.cpp:33-50),
              masked entries zero (cuda/gpu_ops.cu:495-503), times scale; dQ = dS K; dK = dS^T Q
It differs from the C restatement only in summation order and precision (float64 accumulation),
and tests/test_oracle.py pins it against the C oracle at 1e-5. Only tests and bench.py's
after-the-timing verification import it; nothing under dadgpt_b200 does.
"""
from __future__ import annotations

import numpy as np


def attention_unit(q, k, v, dout=None, scale=1.0, block=1024):
    """q, k, v (and dout): [S, D] arrays of ONE (batch, head) unit. Returns (out, lse) or, with
    dout, (out, lse, dq, dk, dv), all float64."""
    q, k, v = (np.asarray(x, np.float64) for x in (q, k, v))
    S, D = q.shape
    out = np.empty((S, D))
    lse = np.empty(S)
    if dout is not None:
        dout = np.asarray(dout, np.float64)
        dq, dk, dv = np.empty((S, D)), np.zeros((S, D)), np.zeros((S, D))
    cols = np.arange(S)
    for r0 in range(0, S, block):
        r1 = min(r0 + block, S)
        n = r1  # keys visible to this block of rows
        s = (q[r0:r1] @ k[:n].T) * scale
        hidden = cols[None, :n] > np.arange(r0, r1)[:, None]
        s[hidden] = -np.inf
        mx = s.max(axis=1, keepdims=True)
        e = np.exp(s - mx)
        sm = e.sum(axis=1, keepdims=True)
        p = e / sm
        out[r0:r1] = p @ v[:n]
        lse[r0:r1] = (mx + np.log(sm))[:, 0]
        if dout is not None:
            g = dout[r0:r1]
            dv[:n] += p.T @ g
            dp = g @ v[:n].T
            ds = p * (dp - (dp * p).sum(axis=1, keepdims=True)) * scale
            dq[r0:r1] = ds @ k[:n]
            dk[:n] += ds.T @ q[r0:r1]
    if dout is None:
        return out, lse
    return out, lse, dq, dk, dv
