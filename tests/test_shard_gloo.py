"""The multi-GPU row split on CPU: two gloo ranks shard a batch's rows the way the GPU path does,
exchange them with the package's own all-gather helper and must reassemble the single-process
result.  Also checks the ownership arithmetic against a brute-force count."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from orca_b200 import shard


def test_ownership_arithmetic():
    for world in (1, 2, 3, 4, 8):
        for n in (0, 1, 7, 8, 9, 2000, 6601):
            counts = [shard.local_count(n, r, world) for r in range(world)]
            assert counts == [len(range(r, n, world)) for r in range(world)]
            assert sum(counts) == n
        rpr = shard.rows_per_rank(6601, world)
        slots = [shard.owner_slot(i, world, rpr) for i in range(6601)]
        assert len(set(slots)) == 6601 and max(slots) < world * rpr


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, b, cap):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rs = np.random.RandomState(0)                     # same data on every rank
        full_l1 = torch.from_numpy(rs.randn(cap, 5).astype(np.float32))   # layer-1 rows in global order
        n1 = cap - 37                                      # rows beyond n1 are garbage on purpose
        rpr = shard.rows_per_rank(cap, world)
        local = torch.full((rpr, 5), float("nan"))
        mine = torch.arange(rank, n1, world)
        local[: len(mine)] = full_l1[mine]
        gathered = shard.all_gather_rows(local).view(world * rpr, 5)
        idx = torch.tensor([shard.owner_slot(i, world, rpr) for i in range(n1)])
        assert torch.equal(gathered[idx], full_l1[:n1])

        # edge-major blocks: [pos | neg] scores and [src | dst | neg] embeddings
        full_scores = torch.from_numpy(rs.rand(2 * b).astype(np.float32))
        n_loc, n_max = shard.local_count(b, rank, world), shard.rows_per_rank(b, world)
        loc = torch.full((2 * n_max,), float("nan"))
        e = torch.arange(rank, b, world)
        loc[:n_loc] = full_scores[e]
        loc[n_loc:2 * n_loc] = full_scores[b + e]
        out = shard.assemble_edges(shard.all_gather_rows(loc), b, 2)
        assert torch.equal(out, full_scores)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("b,cap", [(200, 1260), (7, 50)])
def test_two_rank_exchange_reassembles(b, cap):
    mp.spawn(_worker, args=(2, _free_port(), b, cap), nprocs=2, join=True)


@pytest.mark.parametrize("world,b,cap", [(4, 203, 1270), (3, 10, 64)])
def test_more_ranks_exchange_reassembles(world, b, cap):
    """Row counts that do not divide by the number of ranks, four and three ranks."""
    mp.spawn(_worker, args=(world, _free_port(), b, cap), nprocs=world, join=True)
