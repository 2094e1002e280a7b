"""The (batch x head) partition on two GPUs: every rank builds the lists and runs the sparse pass on its
own units, the outputs are gathered with NCCL, and rank 0 compares the gathered tensor bit for bit
with the single-GPU run of the whole workload.  Skipped on a box with one GPU."""
import os
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def _worker(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from fgattn_tk_cuda_b200 import capi, sharded, synth
    import fgattn_tk_cuda_b200.spattn as spattn
    w = synth.Workload("mg", 1, 6, 1200, 128, "clustered", centroids=8, run=64, tau=1e-3, seed=321)
    total = w.B * w.H

    def run(units):
        q, k, v = synth.make_qkv(w, device="cuda", heads=units)
        idx, cnt, m, l = spattn.mask_utils.qk_block_indexmask_cuda(q, k, w.tau)
        o = torch.empty_like(q)
        capi.sp_attn_blocks_ml(o, q, k, v, idx, cnt, m, l)
        capi.check()
        return o[0], idx[0], cnt[0]

    units = sharded.local_units(total)
    o, idx, cnt = run(units)
    o_all = sharded.all_gather_units(o, total)
    idx_all = sharded.all_gather_units(idx, total)
    cnt_all = sharded.all_gather_units(cnt, total)
    torch.cuda.synchronize()
    if rank == 0:
        o1, idx1, cnt1 = run(range(total))
        ok = torch.equal(o_all, o1) and torch.equal(idx_all, idx1) and torch.equal(cnt_all, cnt1)
        Path(tmp, "result.txt").write_text("ok" if ok else "mismatch")
    dist.destroy_process_group()


def test_two_gpu_partition_and_nccl_gather(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = 29600 + (os.getpid() % 1000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "result.txt").read_text() == "ok"
