"""Process-group bring-up and the global -> per-rank token split.

``init_distributed`` has the contract of the reference's (common.py:51-67): read
RANK / WORLD_SIZE / LOCAL_RANK, bind the GPU, create the NCCL group pinned to that GPU.
Without CUDA it creates a gloo group so the host logic runs as CPU ranks.
"""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist


def init_distributed(backend: str | None = None, timeout_s: float | None = None):
    """Returns ``(group, rank, world_size, local_rank)``.  A single process without torchrun
    variables becomes a world of one."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    use_cuda = torch.cuda.is_available()
    ndev = torch.cuda.device_count() if use_cuda else 1
    local_rank = int(os.environ.get("LOCAL_RANK", rank % max(ndev, 1)))
    if backend is None:
        backend = "nccl" if use_cuda else "gloo"
    if use_cuda:
        torch.cuda.set_device(local_rank)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        kwargs = {}
        if timeout_s is not None:
            kwargs["timeout"] = datetime.timedelta(seconds=timeout_s)
        if backend == "nccl":
            kwargs["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kwargs)
    return dist.group.WORLD, rank, world, local_rank


def local_token_count(global_b: int, rank: int, world: int) -> int:
    """Balanced split: rank r holds B // world tokens, plus one if r < B % world."""
    return global_b // world + (1 if rank < global_b % world else 0)


def all_rank_counts(global_b: int, world: int) -> list[int]:
    return [local_token_count(global_b, r, world) for r in range(world)]
