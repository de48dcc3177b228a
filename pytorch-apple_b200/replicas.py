"""Batch-sharded replicas: one process per GPU, every process with the whole model.

The reference runs on one device (``CUDABackend(device_id=0)``, cuda_backend.py:97-101) and has
no multi-device code.  Images and decode sequences are independent, so the multi-GPU form of
this backend is N copies of the same executor - weights replicated, the batch split into
contiguous shards, no collective on the data path.  The process group (NCCL on GPUs, gloo on
hosts) only carries the barrier that starts a timed region, the gathered results and the max of
the per-rank timings.

Launch with ``python -m torch.distributed.run --nproc-per-node N ...``; each rank calls
``init()`` and builds its executors for ``per_rank_batch`` rows on ``device()``.
"""

from __future__ import annotations

import os
from typing import Any, Callable

import numpy as np

try:
    import torch
    import torch.distributed as dist
except ImportError:  # pragma: no cover
    torch = None
    dist = None


def world() -> tuple[int, int, int]:
    """(rank, world size, local rank) from the launcher's environment (1-process defaults)."""
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def init(backend: str | None = None) -> tuple[int, int, int]:
    """Join the process group when launched with more than one rank; returns ``world()``."""
    rank, size, local = world()
    if size > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        use_cuda = torch.cuda.is_available()
        if use_cuda:
            torch.cuda.set_device(local)
        dist.init_process_group(backend or ("nccl" if use_cuda else "gloo"), rank=rank, world_size=size)
    return rank, size, local


def shard_bounds(n_items: int, size: int, rank: int) -> tuple[int, int]:
    """Rows [lo, hi) of a batch of ``n_items`` served by ``rank``: contiguous, sizes differ by at most one."""
    if not 0 <= rank < size:
        raise ValueError(f"rank {rank} outside a group of {size}")
    q, r = divmod(n_items, size)
    lo = rank * q + min(rank, r)
    return lo, lo + q + (1 if rank < r else 0)


def shard_inputs(inputs: dict[str, Any], batched: set[str], n_items: int, size: int, rank: int) -> dict[str, Any]:
    """This rank's rows of every batched input (axis 0); other inputs are passed whole."""
    lo, hi = shard_bounds(n_items, size, rank)
    return {k: (v[lo:hi] if k in batched else v) for k, v in inputs.items()}


def gather_rows(local: np.ndarray, size: int, rank: int, root: int = 0) -> np.ndarray | None:
    """Concatenate every rank's result rows on ``root`` (in rank order, i.e. in batch order); ``None`` elsewhere.
    Results are small next to the work that produced them (token ids, logits of a shard); they travel as host objects."""
    if size == 1:
        return local
    parts: list[Any] | None = [None] * size if rank == root else None
    dist.gather_object(local, parts, dst=root)
    return np.concatenate(parts, axis=0) if rank == root else None


def run_sharded(step: Callable[[dict[str, Any]], np.ndarray], inputs: dict[str, Any], batched: set[str], n_items: int) -> np.ndarray | None:
    """One sharded call: ``step`` (this rank's executor, compiled for its shard's batch) on this rank's
    rows, results gathered on rank 0.  Every rank must call it; no rank reads another rank's inputs."""
    rank, size, _ = world()
    return gather_rows(step(shard_inputs(inputs, batched, n_items, size, rank)), size, rank)


def max_over_ranks(values, device=None) -> list[float]:
    """Element-wise MAX of per-rank timings: a sharded job is as slow as its slowest replica."""
    _, size, _ = world()
    if size <= 1:
        return [float(v) for v in values]
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t]
