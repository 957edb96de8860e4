"""Process-group plumbing: one process per GPU launched by torchrun (RANK / LOCAL_RANK / WORLD_SIZE /
MASTER_*), NCCL on GPUs and gloo on CPU. Replaces the MPI + tutel bootstrap of the reference
(mix_moe/csrc/mix_moe.h:58-70, mix_moe/mix_moe/examples/mix_moe_ddp.py:33-35)."""
from __future__ import annotations

import datetime
import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist


def env_rank() -> Tuple[int, int, int]:
    """(rank, local_rank, world_size) from the launcher's environment; (0, 0, 1) when not launched."""
    return (int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)),
            int(os.environ.get("WORLD_SIZE", 1)))


def init_distributed(backend: Optional[str] = None, timeout_s: float = 600.0) -> Tuple[int, int, int]:
    """Initialise the default process group if WORLD_SIZE > 1 (or already set up) and pick the device."""
    rank, local_rank, world = env_rank()
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local_rank % torch.cuda.device_count())
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        backend = backend or ("nccl" if use_cuda else "gloo")
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group(backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return rank, local_rank, world


def group_size(group=None) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


def group_rank(group=None) -> int:
    return dist.get_rank(group) if dist.is_initialized() else 0


def make_ep_dp_groups(ep_size: int):
    """Split the world into expert-parallel groups of ``ep_size`` consecutive ranks and the
    data-parallel groups that connect equal positions of those groups ("EP=8, DP over the rest").
    Returns (ep_group, dp_group); every rank must call this."""
    if not dist.is_initialized():
        return None, None
    world, rank = dist.get_world_size(), dist.get_rank()
    if world % ep_size:
        raise ValueError("world size must be a multiple of ep_size")
    ep_group = dp_group = None
    for g in range(world // ep_size):
        ranks = list(range(g * ep_size, (g + 1) * ep_size))
        grp = dist.new_group(ranks)
        if rank in ranks:
            ep_group = grp
    for p in range(ep_size):
        ranks = list(range(p, world, ep_size))
        grp = dist.new_group(ranks)
        if rank in ranks:
            dp_group = grp
    return ep_group, dp_group


def get_torch_default_comm():
    """The default process group (kept for users of mix_moe/mix_moe/utils.py:7-29)."""
    return dist.group.WORLD if dist.is_initialized() else None


def get_rank_0_in_comm(comm=None) -> int:
    """Global rank of the first member of ``comm`` (mix_moe/mix_moe/utils.py:32-37)."""
    if not dist.is_initialized():
        return 0
    return dist.get_global_rank(comm, 0) if comm is not None else 0


def max_over_ranks(value: float, group=None) -> float:
    if not dist.is_initialized():
        return float(value)
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
