"""N > 1 host logic on CPU: two gloo ranks, each a replica with its own shard of the
requests; the job's time is the slowest rank's, the job's throughput counts all ranks."""

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _worker(rank: int, world: int, port: int, out):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "pytorch-apple_b200"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench

    # every rank serves its own sequences: shard ids differ, no data-path collective
    shard = list(range(rank * 4, rank * 4 + 4))
    my_ms = [10.0 + 5.0 * rank, 20.0 - 3.0 * rank]
    dist.barrier()
    ms, e2e = bench.max_over_ranks(my_ms, world)
    out[rank] = (shard, ms, e2e, bench.whole_job_throughput(world, 4, 8, ms))
    dist.barrier()
    dist.destroy_process_group()


def test_two_replicas_report_max_time_and_summed_work():
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, 29731, out), nprocs=world, join=True)
        res = dict(out)
    assert res[0][0] == [0, 1, 2, 3] and res[1][0] == [4, 5, 6, 7]
    for r in range(world):
        assert res[r][1] == 15.0 and res[r][2] == 20.0            # max over ranks, on every rank
        assert abs(res[r][3] - world * 4 * 8 / 0.015) < 1e-6       # whole-job units / slowest time


def test_single_rank_is_identity():
    sys.path.insert(0, str(ROOT))
    import bench

    assert bench.max_over_ranks([3.5, 1.0], 1) == [3.5, 1.0]
    assert bench.whole_job_throughput(1, 64, 10, 100.0) == 6400.0
