"""Host logic of the (batch x head) partition, run as two gloo ranks on the CPU."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _worker(rank, world, port, total, tmp):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fgattn_tk_cuda_b200 import sharded, synth
    w = synth.Workload("t", 1, total, 96, 64, "clustered", centroids=4, run=32, tau=1e-3, seed=9)
    units = sharded.local_units(total)
    q, k, v = synth.make_qkv(w, heads=units)
    # stand-in for the per-unit kernel: anything that is a function of the unit's own q, k, v
    local = (q[0].float() + 2 * k[0].float() - v[0].float())
    full = sharded.all_gather_units(local, total)
    idx_local = torch.tensor([[u, u * u] for u in units], dtype=torch.int32).reshape(len(units), 2)
    idx_full = sharded.all_gather_units(idx_local, total)
    torch.save({"full": full, "idx": idx_full, "units": list(units)}, f"{tmp}/r{rank}.pt")
    dist.destroy_process_group()


@pytest.mark.parametrize("total", [4, 5])
def test_two_rank_partition_and_gather(tmp_path, total):
    from fgattn_tk_cuda_b200 import synth
    port = 29500 + (os.getpid() % 2000) + total
    mp.spawn(_worker, args=(2, port, total, str(tmp_path)), nprocs=2, join=True)
    w = synth.Workload("t", 1, total, 96, 64, "clustered", centroids=4, run=32, tau=1e-3, seed=9)
    q, k, v = synth.make_qkv(w)
    want = q[0].float() + 2 * k[0].float() - v[0].float()
    seen = []
    for r in range(2):
        d = torch.load(f"{tmp_path}/r{r}.pt")
        assert torch.equal(d["full"], want)          # shards reproduce the single-process tensor exactly
        assert d["idx"][:, 0].tolist() == list(range(total))
        seen += d["units"]
    assert sorted(seen) == list(range(total))         # every unit owned exactly once


def test_shard_heads_properties():
    from fgattn_tk_cuda_b200.synth import shard_heads
    for total in (1, 7, 32, 96, 512):
        for world in (1, 2, 4, 8):
            parts = [shard_heads(total, world, r) for r in range(world)]
            flat = [u for p in parts for u in p]
            assert flat == list(range(total))
            assert max(len(p) for p in parts) - min(len(p) for p in parts) <= 1
