"""CPU: the multi-rank path (unit sharding + verification all-gather) on two gloo ranks."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dadgpt_b200.sharding import shard_units

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_units_cover_everything_once():
    for total in (0, 1, 7, 192, 193):
        for world in (1, 2, 3, 8):
            shards = [shard_units(total, world, r) for r in range(world)]
            assert sum(s.count for s in shards) == total
            pos = 0
            for s in shards:
                assert s.unit0 == pos
                pos += s.count
            assert max(s.count for s in shards) - min(s.count for s in shards) <= 1
    with pytest.raises(ValueError):
        shard_units(4, 2, 2)


def _worker(rank, world, port, total, tmp):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from dadgpt_b200.sharding import all_gather_units, shard_units as su
    from oracle.oracle import Oracle
    ora = Oracle()
    rng = np.random.default_rng(3)
    S, D = 40, 16
    q, k, v = (rng.standard_normal((total, S, D), dtype=np.float32) for _ in range(3))
    sh = su(total, world, rank)
    # each rank computes only its units; unit0 keeps the dropout mask global
    out, _ = ora.forward(q[sh.units], k[sh.units], v[sh.units], 0.25, rate=0.1, seed=42,
                         unit0=sh.unit0, threads=2)
    full = all_gather_units(torch.from_numpy(out), total)
    whole, _ = ora.forward(q, k, v, 0.25, rate=0.1, seed=42, threads=2)
    ok = np.array_equal(full.numpy(), whole)
    with open(os.path.join(tmp, f"rank{rank}.txt"), "w") as f:
        f.write("ok" if ok else "mismatch")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("total", [6, 5])
def test_two_gloo_ranks_reassemble_the_unsharded_result(tmp_path, oracle, total):
    port = 29500 + (os.getpid() + total) % 2000
    mp.spawn(_worker, args=(2, port, total, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"
