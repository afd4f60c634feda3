"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch


def dev_f32(x, dev):
    return torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(dev)


def dev_bf16(x, dev):
    """fp32 numpy -> bf16 device tensor (round to nearest even) and its fp32 host upcast."""
    t = torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(dev).to(torch.bfloat16)
    return t, t.float().cpu().numpy()


def rel_l2(got, want):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    # A gradient that is exactly zero in the reference (S = 1: dS = p * (dp - delta) is pure
    # rounding noise) cannot be judged by a ratio; differences below 1e-6 absolute count as equal.
    if np.abs(got - want).max() < 1e-6:
        return 0.0
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


def max_abs(got, want):
    return float(np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64)).max())
