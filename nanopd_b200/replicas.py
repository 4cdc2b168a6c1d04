"""Batch sharding of decode work across GPU replicas (one process per GPU).

Decode sequences are independent, so a decode batch shards across replicas with NO
data-path collective — the layout the reference uses when it builds one full model replica
per worker GPU (nanoPD/router/central_scheduler.py:101-117).  ``torch.distributed`` is used
only for plumbing: a barrier around timed regions, the max of a per-rank time and the sum
of per-rank work.
"""
from __future__ import annotations

import os
from typing import List, Sequence

import torch
import torch.distributed as dist

from .workloads import shard_sequences


def env_world():
    """(rank, local_rank, world_size) from the torchrun environment, (0, 0, 1) when absent."""
    return (int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)),
            int(os.environ.get("WORLD_SIZE", 1)))


def init_process_group(backend: str):
    rank, local_rank, world = env_world()
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group(backend=backend, rank=rank, world_size=world)
    return rank, local_rank, world


def barrier():
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


_host_group = None


def host_barrier(timeout_s: float = 1800.0):
    """A barrier that waits on the HOST (a gloo group over the same ranks).  For phases in which one rank drives
    several GPUs for a long time while the others wait: an NCCL barrier would park a spinning kernel on every
    waiting rank's GPU, next to the kernels the working rank launches there."""
    global _host_group
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return
    if _host_group is None:
        import datetime
        _host_group = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))
    dist.barrier(group=_host_group)


def max_over_ranks(value: float, device="cpu") -> float:
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, device="cpu") -> float:
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def shard_batch_rows(tensors: Sequence[torch.Tensor], rank: int, world_size: int) -> List[torch.Tensor]:
    """Rows [lo, hi) of every per-sequence tensor for this replica (a contiguous batch shard)."""
    n = tensors[0].size(0)
    r = shard_sequences(n, rank, world_size)
    return [t[r.start:r.stop] for t in tensors]


def gather_rows(local: torch.Tensor, world_size: int) -> torch.Tensor:
    """All replicas' output rows, in rank order (used by tests to compare with a 1-replica run)."""
    if world_size == 1:
        return local
    sizes = [torch.zeros(1, dtype=torch.int64) for _ in range(world_size)]
    dist.all_gather(sizes, torch.tensor([local.size(0)], dtype=torch.int64))
    maxn = int(max(int(s) for s in sizes))
    pad = torch.zeros((maxn,) + tuple(local.shape[1:]), dtype=local.dtype)
    pad[:local.size(0)] = local
    bufs = [torch.zeros_like(pad) for _ in range(world_size)]
    dist.all_gather(bufs, pad)
    return torch.cat([b[:int(s)] for b, s in zip(bufs, sizes)])
