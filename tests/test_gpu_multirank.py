"""GPU, two ranks (skipped on a single-GPU box): each rank computes its contiguous range of
(batch x head) units with the CUDA kernels, the results are all-gathered over NCCL, and rank 0
compares them with the same computation done unsharded on one GPU. dK, dV, out and lse must be
bit-identical (a unit's result does not depend on which rank computed it, nor does its dropout
mask, thanks to unit0); dQ of the single-pass backward is summed in arrival order and is compared
at 1e-2 relative L2. No collective runs inside the attention path itself."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _compute(dad, ws_bytes, q, k, v, do, scale, unit0, rate):
    BH, S, D = q.shape
    out, lse = torch.empty_like(q), torch.empty(BH, S, device=q.device)
    kw = dict(rate=rate, seed=42, offset=0, unit0=unit0)
    dad.gpu_flash_attention_forward_bf16(out, lse, q, k, v, BH, S, D, scale, **kw)
    grads = [torch.empty_like(q) for _ in range(3)]
    ws = torch.empty(ws_bytes(BH, S, D), dtype=torch.uint8, device=q.device)
    dad.gpu_flash_attention_backward_bf16(*grads, ws, do, out, lse, q, k, v, BH, S, D, scale, **kw)
    return [out, lse] + grads


def _worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import dadgpt_b200 as dad
    from dadgpt_b200.attention import device_status, flash_backward_bf16_workspace_bytes
    from dadgpt_b200.sharding import all_gather_units, shard_units
    ok = True
    for D, S, total, rate in ((64, 300, 10, 0.0), (64, 257, 7, 0.1), (128, 200, 6, 0.0)):
        g = torch.Generator().manual_seed(1000 + D + S)   # the same tensors on every rank
        full = [(torch.randn(total, S, D, generator=g) * 0.5).to(torch.bfloat16) for _ in range(4)]
        sh = shard_units(total, world, rank)
        mine = [t[sh.units].to(dev) for t in full]
        res = _compute(dad, flash_backward_bf16_workspace_bytes, *mine, D ** -0.5, sh.unit0, rate)
        gathered = [all_gather_units(t, total) for t in res]
        if rank == 0:
            whole = _compute(dad, flash_backward_bf16_workspace_bytes, *[t.to(dev) for t in full],
                             D ** -0.5, 0, rate)
            for name, a, b in zip(("out", "lse", "dq", "dk", "dv"), gathered, whole):
                if name == "dq":
                    d = (a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30)
                    ok &= bool(d <= 1e-2)
                else:
                    ok &= bool(torch.equal(a, b))
        ok &= device_status() == 0
    with open(os.path.join(tmp, f"rank{rank}.txt"), "w") as f:
        f.write("ok" if ok else "mismatch")
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reassemble_the_unsharded_result(cuda, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"
