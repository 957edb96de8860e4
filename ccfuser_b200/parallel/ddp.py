"""Data parallelism around expert parallelism: expert parameters live on one rank of the expert-parallel
group and must not be all-reduced; everything else (attention, dense FFNs, embeddings, routers) is replicated.

Same convention as the reference: expert parameters carry ``skip_allreduce = True``
(mix_moe/mix_moe/transformer.py:454-456) and their names go into DDP's ignore list
(mix_moe/mix_moe/examples/mix_moe_ddp.py:139-152, examples/models/moe_gpt.py:1200-1203).
"""
from __future__ import annotations

import os
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
    # bucket size of the gradient all-reduce (MB): NVSwitch gives every message full bandwidth, so a bucket is sized for
    # launch count and for overlap with the backward pass, not for a link count (GPT-MoE 24 L on 4 GPUs: 121.1 ms per
    # step with torch's 25 MB, 119.4 ms with 100 MB, 119.8 ms with 400 MB)
    kw.setdefault("bucket_cap_mb", int(os.environ.get("CCFUSER_DDP_BUCKET_MB", "100")))
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


def reduce_expert_grads(model: nn.Module, dp_group=None, scale: float = None):
    """Gradients of the expert parameters when the expert-parallel group is smaller than the job ("EP inside a node, DP
    over the rest", utils/dist.py: make_ep_dp_groups): every data-parallel replica of an expert has seen only the
    tokens of its own expert-parallel group, so the replicas' gradients are summed over ``dp_group`` (the ranks that
    hold the same experts). ``scale`` then multiplies the result; ``1 / world_size`` gives the expert parameters the
    same mean-over-all-ranks convention that DistributedDataParallel applies to the replicated ones (without it an
    expert's gradient is the plain sum over the ranks whose tokens it served, which is what the reference's ignore-list
    set-up leaves, mix_moe/mix_moe/examples/mix_moe_ddp.py:139-152)."""
    grads = [p.grad for p in model.parameters() if p.grad is not None and getattr(p, "skip_allreduce", False)]
    if not grads:
        return
    replicas = dist.get_world_size(dp_group) if (dist.is_initialized() and dp_group is not None) else 1
    if replicas > 1:
        # one flat buffer per dtype keeps this at one or two collectives
        by_dtype = {}
        for g in grads:
            by_dtype.setdefault(g.dtype, []).append(g)
        for gs in by_dtype.values():
            flat = torch._utils._flatten_dense_tensors(gs)
            dist.all_reduce(flat, group=dp_group)
            if scale is not None:
                flat.mul_(scale)
            for g, f in zip(gs, torch._utils._unflatten_dense_tensors(flat, gs)):
                g.copy_(f)
    elif scale is not None:
        torch._foreach_mul_(grads, scale)
