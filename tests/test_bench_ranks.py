"""The multi-rank bookkeeping of bench.py on CPU: two gloo ranks, max-over-ranks
timing and the whole-job value (replicas: no data-path collective)."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _rank(rank: int, world: int, port: int, results) -> None:
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    mine = [10.0 + rank, 3.0 - rank]            # rank 1 is slower on the first, faster on the second
    results[rank] = bench.max_over_ranks(mine)
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_report_the_slowest_time():
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_rank, args=(2, 29613, results), nprocs=2, join=True)
    assert results[0] == [11.0, 3.0] and results[1] == [11.0, 3.0]


def test_job_value_counts_every_replica():
    sys.path.insert(0, str(ROOT))
    import bench
    assert bench.max_over_ranks([1.5, 2.5]) == [1.5, 2.5]          # no process group: identity
    assert bench.job_value(world=4, batch=2, steps=10, seconds=0.5) == 160.0
