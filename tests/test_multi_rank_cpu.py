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


def _replica_worker(rank: int, world: int, port: int, out):
    """A real sharded inference: ResNet-18 on a batch of 6 images, 2 replicas of 3 images each, through
    the whole host pipeline (the kernel library replaced by the host stand-in), gathered on rank 0."""
    for p in (ROOT / "tests", ROOT, ROOT / "pytorch-apple_b200"):
        sys.path.insert(0, str(p))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    import numpy as np

    import model_zoo as mz
    import replicas
    from cuda_compiler import compile_subgraph, is_cuda_op_supported
    from cuda_runtime import CUDABackend, native
    from fake_b200nn import FakeLibrary
    from ir_export import extract_ir
    from npu_compiler import partition
    from npu_runtime import DAGExecutor

    native.install_test_library(FakeLibrary(), "cpu")
    assert replicas.init("gloo") == (rank, world, rank)
    n_items = 6
    lo, hi = replicas.shard_bounds(n_items, world, rank)
    m = mz.resnet(18, seed=0)
    x = torch.randn(n_items, 3, 64, 64, generator=torch.Generator().manual_seed(1))     # same on every rank: the "request queue"
    ir = extract_ir(m, (x[lo:hi],), "resnet18")                                           # this rank's executor serves hi - lo images
    dag = DAGExecutor(partition(ir, is_cuda_op_supported), CUDABackend(), compile_subgraph)
    dag.load_weights(mz.state_dict_numpy(m.state_dict()))
    name = ir["graph_outputs"][0]["name"]
    step = lambda shard: dag.execute({"x": shard["x"]})[name].to_numpy().astype(np.float32)
    logits = replicas.run_sharded(step, {"x": x.numpy()}, {"x"}, n_items)
    slowest = replicas.max_over_ranks([1.0 + rank])
    if rank == 0:
        with torch.no_grad():
            want = m(x).numpy()
        out["err"] = float(np.abs(logits - want).max())
        out["shape"] = tuple(logits.shape)
        out["top1"] = bool((logits.argmax(-1) == want.argmax(-1)).all())
    else:
        assert logits is None
    out[f"slowest{rank}"] = slowest[0]
    dist.barrier()
    dist.destroy_process_group()


def test_two_replicas_serve_one_batch_through_the_whole_pipeline():
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_replica_worker, args=(world, 29741, out), nprocs=world, join=True)
        res = dict(out)
    assert res["shape"] == (6, 1000) and res["err"] <= 1e-1 and res["top1"]
    assert res["slowest0"] == res["slowest1"] == 2.0


def test_shard_bounds_cover_the_batch_in_order():
    sys.path.insert(0, str(ROOT / "pytorch-apple_b200"))
    import replicas

    for n, size in ((64, 8), (6, 4), (3, 8), (256, 2)):
        parts = [replicas.shard_bounds(n, size, r) for r in range(size)]
        assert parts[0][0] == 0 and parts[-1][1] == n and all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
        assert max(hi - lo for lo, hi in parts) - min(hi - lo for lo, hi in parts) <= 1
