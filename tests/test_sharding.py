"""Batch sharding across ranks: pure host logic, checked with two gloo ranks on CPU."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from libmolgrid_b200.sharding import shard_bounds, my_slice


def test_bounds_partition_and_balance():
    rng = np.random.default_rng(0)
    for batch, world in ((50, 1), (50, 2), (50, 8), (1024, 8), (3, 8), (0, 4), (7, 7)):
        n = rng.integers(2000, 4001, batch)
        b = shard_bounds(n, world)
        assert len(b) == world and b[0][0] == 0 and b[-1][1] == batch
        assert all(b[i][1] == b[i + 1][0] for i in range(world - 1))       # contiguous, disjoint, complete
        assert all(s <= e for s, e in b)
        if batch >= 8 * world:
            work = [float((n[s:e] + 1200).sum()) for s, e in b]
            assert max(work) / (sum(work) / world) < 1.15
    with pytest.raises(ValueError):
        shard_bounds([1, 2], 0)


def _rank_main(rank, world, port, n_atoms, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    s, e = my_slice(n_atoms, rank, world)
    # each rank "grids" its own examples; here the stand-in result is the atom count per example
    mine = torch.zeros(len(n_atoms), dtype=torch.int64)
    mine[s:e] = torch.as_tensor(n_atoms[s:e])
    owner = torch.zeros(len(n_atoms), dtype=torch.int64)
    owner[s:e] = 1
    # verification only (not part of the data path): every example is owned exactly once
    dist.all_reduce(mine)
    dist.all_reduce(owner)
    if rank == 0:
        out.put((mine.tolist(), owner.tolist()))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_cover_the_batch_once():
    n_atoms = np.random.default_rng(1).integers(2000, 4001, 50)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, n_atoms, out)) for r in range(2)]
    for p in procs:
        p.start()
    mine, owner = out.get(timeout=120)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert owner == [1] * 50
    assert mine == n_atoms.tolist()
