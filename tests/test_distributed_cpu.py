"""The multi-GPU host logic on CPU ranks (gloo, world size 2): partition, shards, the one-off
replication of B, max-over-ranks timing.  The per-rank product is done by the CPU oracle here --
the point is the plumbing around it, which is the same code the GPU bench runs over NCCL."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from csrspmm_b200 import distributed as D, generators as G

    # rank 0 owns the problem; sizes, A and B are replicated once, as bench.py does over NCCL
    if rank == 0:
        p = G.make("cfg3_powerlaw", scale=512)
        sizes = torch.tensor([p.M, p.Kd, p.Nd, p.nnz])
    else:
        p, sizes = None, torch.zeros(4, dtype=torch.int64)
    dist.broadcast(sizes, 0)
    M, Kd, Nd, nnz = sizes.tolist()
    row_ptr = torch.from_numpy(p.row_ptr) if rank == 0 else torch.empty(M + 1, dtype=torch.int32)
    col_idx = torch.from_numpy(p.col_idx) if rank == 0 else torch.empty(nnz, dtype=torch.int32)
    values = torch.from_numpy(p.values) if rank == 0 else torch.empty(nnz, dtype=torch.float32)
    B = torch.from_numpy(p.B) if rank == 0 else torch.empty((Kd, Nd), dtype=torch.float32)
    for t in (row_ptr, col_idx, values, B):
        D.replicate(t, 0)

    bounds = D.partition_rows(row_ptr, world)
    sh = D.take_shard(row_ptr, col_idx, values, bounds, rank)
    assert sh.row_ptr[0] == 0 and int(sh.row_ptr[-1]) == sh.nnz
    C_shard = oracle.spmm(sh.row_ptr.numpy(), sh.col_idx.numpy(), sh.values.numpy(), B.numpy())

    # C stays sharded; the test alone gathers it to compare with the unsharded product
    np.save(Path(out_dir) / f"c{rank}.npy", C_shard)
    np.save(Path(out_dir) / f"b{rank}.npy", np.asarray(bounds))
    t_job = D.max_over_ranks(1.0 + rank, "cpu")  # slowest rank defines the step time
    total_nnz = D.sum_over_ranks(float(sh.nnz), "cpu")
    assert t_job == float(world) and total_nnz == float(nnz)
    dist.barrier()
    if rank == 0:
        full = oracle.spmm(p.row_ptr, p.col_idx, p.values, p.B)
        got = np.concatenate([np.load(Path(out_dir) / f"c{r}.npy") for r in range(world)])
        assert np.array_equal(got, full)
        assert all(np.array_equal(np.load(Path(out_dir) / f"b{r}.npy"), bounds) for r in range(world))
        assert D.partition_imbalance(p.row_ptr, bounds) < 1.1
    dist.destroy_process_group()


def test_row_sharded_product_world_size_2(tmp_path):
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
