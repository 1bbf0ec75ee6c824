"""The sharded end-to-end path on real GPUs: one process per GPU over NCCL (skipped on a box with one
GPU).  Every rank holds, in pinned host memory, its row block of A and its slice of B's rows; the
pipeline uploads, all-gathers B panel by panel, multiplies and downloads.  Checked against the CPU
oracle on the rank's own rows."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, panels, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import oracle
    from csrspmm_b200 import distributed as D, generators as G

    p = G.make("cfg3_powerlaw", scale=64, Nd=256)  # same seed on every rank: same problem, built on the host
    assert p.Kd % world == 0
    bounds = D.partition_rows(p.row_ptr, world)
    sh = D.take_shard(torch.from_numpy(p.row_ptr), torch.from_numpy(p.col_idx), torch.from_numpy(p.values), bounds, rank)
    sh.row_ptr, sh.col_idx, sh.values = sh.row_ptr.pin_memory(), sh.col_idx.pin_memory(), sh.values.pin_memory()
    sl = p.Kd // world
    hB = torch.from_numpy(p.B[rank * sl:(rank + 1) * sl].copy()).pin_memory()
    runner = D.ShardedHostSpmm(sh, hB, p.Kd, torch.device("cuda", rank), panels=panels)
    assert len(runner.panels) == panels
    f64, mag = oracle.spmm_f64(sh.row_ptr.numpy(), sh.col_idx.numpy(), sh.values.numpy(), p.B, threads=2)
    ok = True
    for _ in range(2):
        runner.C_host.fill_(float("nan"))
        got = runner.run().numpy()
        ok = ok and bool((np.abs(got - f64) <= 1e-5 * mag + 1e-6).all())
    t = D.max_over_ranks(float(rank), torch.device("cuda", rank))
    ok = ok and t == float(world - 1)
    (Path(out_dir) / f"ok{rank}").write_text("1" if ok else "0")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("panels", [1, 2])
def test_sharded_host_pipeline_over_nccl(cuda_lib, tmp_path, panels):
    world = min(torch.cuda.device_count(), 2)
    if world < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(world, _free_port(), panels, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").read_text() == "1" for r in range(world))
