"""Generates tests/golden/*.npz by running the REFERENCE's own host ops.

Run where the reference tree is present ($DADGPT_REFERENCE_DIR, or a directory named
`reference` beside this repository):

    python tests/golden/make_golden.py

It builds oracle/_ref/libdadref_host.so from the reference's src/tensor_ops.cpp and
src/backward.cpp (see oracle/Makefile) and drives them in the call order of the reference's
materialized attention (oracle/ref_compose.cpp). Inputs are regenerated from seeds by
dadgpt_b200.workloads, so only outputs are stored. The dropout masks fed to the reference ops
come from the oracle's Philox (the reference has no host dropout); on a GPU they are checked
against the reference's dropout kernel by tests/test_gpu_dropout.py.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from dadgpt_b200 import workloads as W  # noqa: E402
from oracle.oracle import Oracle, RefHost, build_oracle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    build_oracle()
    ref, ora = RefHost(), Oracle()

    # C1: the tiny preset on the host path, fp32, no dropout (D=16 as configured, and the
    # preset's real head size 32).
    for shape in (W.TINY, W.TINY_D32):
        q, k, v = W.qkv(shape)
        out = ref.forward(q, k, v, shape.scale)
        rng = np.random.default_rng(100 + shape.D)
        dout = rng.standard_normal(q.shape, dtype=np.float32)
        dq, dk, dv = ref.backward(dout, q, k, v, shape.scale)
        np.savez_compressed(os.path.join(HERE, f"{shape.name}.npz"), out=out, dq=dq, dk=dk, dv=dv,
                            dout_seed=100 + shape.D)

    # Ragged length of the reference's FusedAttentionMatchesMaterialized test (S=70, d_head 64),
    # with and without dropout (rate 0.3 as in FullModelGradientCheckWithDropout).
    rng = np.random.default_rng(7)
    BH, S, D = 4, 70, 64
    q, k, v, dout = (rng.standard_normal((BH, S, D), dtype=np.float32) for _ in range(4))
    scale = D ** -0.5
    out = ref.forward(q, k, v, scale)
    dq, dk, dv = ref.backward(dout, q, k, v, scale)
    mask = ora.dropout_mask(BH * S * S, 0.3, 42).reshape(BH, S, S)
    out_d = ref.forward(q, k, v, scale, rate=0.3, mask=mask)
    dq_d, dk_d, dv_d = ref.backward(dout, q, k, v, scale, rate=0.3, mask=mask)
    np.savez_compressed(os.path.join(HERE, "ragged_S70_D64.npz"), seed=7, out=out, dq=dq, dk=dk,
                        dv=dv, out_drop=out_d, dq_drop=dq_d, dk_drop=dk_d, dv_drop=dv_d,
                        rate=0.3, drop_seed=42)

    # Decode on the reference cache layout [H,max_len,D], a few positions.
    rng = np.random.default_rng(11)
    H, L, D = 4, 48, 32
    kc, vc = (rng.standard_normal((H, L, D), dtype=np.float32) for _ in range(2))
    qs = rng.standard_normal((3, H, D), dtype=np.float32)
    lens = np.array([1, 17, 48], np.int32)
    outs = np.stack([ref.decode(qs[i], kc, vc, int(lens[i]), D ** -0.5) for i in range(3)])
    np.savez_compressed(os.path.join(HERE, "decode_H4_L48_D32.npz"), seed=11, lens=lens, out=outs)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
