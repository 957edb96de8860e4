"""Data parallelism around expert parallelism: expert parameters live on one rank of the expert-parallel
group and must not be all-reduced; everything else (attention, dense FFNs, embeddings, routers) is replicated.

Same convention as the reference: expert parameters carry ``skip_allreduce = True``
(mix_moe/mix_moe/transformer.py:454-456) and their names go into DDP's ignore list
(mix_moe/mix_moe/examples/mix_moe_ddp.py:139-152, examples/models/moe_gpt.py:1200-1203).
"""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist
import torch.nn as nn


def expert_param_names(model: nn.Module) -> List[str]:
    return [n for n, p in model.named_parameters() if getattr(p, "skip_allreduce", False)]


def add_param_to_skip_allreduce(model: nn.Module) -> List[str]:
    """Record the tagged parameter names where torch DDP looks for parameters to ignore."""
    names = expert_param_names(model)
    torch.nn.parallel.DistributedDataParallel._set_params_and_buffers_to_ignore_for_model(model, names)
    return names


def wrap_ddp(model: nn.Module, process_group=None, **kw):
    """DistributedDataParallel over the replicated parameters only. With one process returns the model."""
    if not dist.is_initialized() or dist.get_world_size(process_group) == 1:
        return model
    add_param_to_skip_allreduce(model)
    dev = next(model.parameters()).device
    ids = [dev.index] if dev.type == "cuda" else None
    kw.setdefault("gradient_as_bucket_view", True)
    return torch.nn.parallel.DistributedDataParallel(model, device_ids=ids, process_group=process_group, **kw)


def allreduce_replicated_grads(model: nn.Module, group=None, average: bool = True):
    """Manual alternative to DDP: one flat all-reduce over the gradients of the replicated parameters."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    grads = [p.grad for p in model.parameters() if p.grad is not None and not getattr(p, "skip_allreduce", False)]
    if not grads:
        return
    flat = torch._utils._flatten_dense_tensors(grads)
    dist.all_reduce(flat, group=group)
    if average:
        flat.div_(dist.get_world_size(group))
    for g, f in zip(grads, torch._utils._unflatten_dense_tensors(flat, grads)):
        g.copy_(f)
