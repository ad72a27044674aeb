"""CPU, world size 2 over gloo: the host side of the multi-GPU modes -- partition arithmetic,
the all-gather that reassembles head-sharded attention outputs, and max-over-ranks timing."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from packkv_b200 import parallel


def test_partition_math():
    assert parallel.partition(8, 0, 2) == (0, 4) and parallel.partition(8, 1, 2) == (4, 8)
    assert [parallel.partition(8, r, 8) for r in range(8)] == [(r, r + 1) for r in range(8)]
    assert parallel.q_heads_of(2, 4, 4) == (8, 16)
    with pytest.raises(ValueError):
        parallel.partition(8, 0, 3)
    with pytest.raises(ValueError):
        parallel.partition(8, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, Hq, D = 3, 8, 128
        full = torch.arange(B * Hq * D, dtype=torch.float32).view(B, Hq, D)
        lo, hi = parallel.partition(Hq, rank, world)
        got = parallel.gather_heads(full[:, lo:hi].clone())
        ok = torch.equal(got, full)
        slowest = parallel.max_over_ranks(10.0 + rank, torch.device("cpu"))
        results[rank] = (ok, slowest)
    finally:
        dist.destroy_process_group()


def test_gather_heads_and_timing_world2():
    world, port = 2, _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert all(results[r][0] for r in range(world))
        assert all(results[r][1] == 11.0 for r in range(world))
