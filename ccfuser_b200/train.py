"""Training step used by the examples and the benchmark: host batch in, loss out.

``TrainStep.step(ids, labels)`` takes pinned host tensors, copies them to the device, runs forward,
backward, the data-parallel all-reduce of the replicated parameters and the optimizer, and returns the
loss as a Python float (one device-to-host read). The reference's loops do the same by hand
(mix_moe/mix_moe/examples/models/moe_gpt_ddp.py:344-381, plain SGD in mix_moe/mix_moe/examples/mix_moe_ddp.py:155).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .parallel.ddp import allreduce_replicated_grads, reduce_expert_grads, wrap_ddp


class TrainStep:
    """One optimisation step as a callable object: forward, backward, gradient reductions, optimizer; see the module docstring."""
    def __init__(self, model: nn.Module, lr: float = 1e-3, optimizer: str = "sgd", dp_group=None,
                 use_ddp: bool = True, aux_loss: bool = False, expert_dp_group=None, mean_expert_grads: bool = False,
                 fuse_expert_sgd: bool = False):
        """``dp_group``: ranks over which the replicated parameters are averaged (default: all). ``expert_dp_group``:
        ranks that hold replicas of this rank's experts (second value of ``make_ep_dp_groups``) when the expert-parallel
        group is smaller than the job. ``mean_expert_grads``: scale expert gradients by 1 / world size so that they
        follow the same mean-over-ranks convention as the replicated parameters. ``fuse_expert_sgd`` (plain SGD, fused
        MoE layers): expert weight matrices are updated inside the backward pass (``MoELayer.fuse_sgd``: all of them on
        single-rank layers, the second projection on layers that span ranks) with the optimizer's current learning rate
        and weight decay."""
        self.raw_model = model
        self.dp_group = dp_group
        self.expert_dp_group = expert_dp_group
        self.mean_expert_grads = mean_expert_grads
        self.distributed = dist.is_initialized() and dist.get_world_size(dp_group) > 1
        self.use_ddp = use_ddp and self.distributed
        self.model = wrap_ddp(model, dp_group) if self.use_ddp else model
        params = [p for p in model.parameters() if p.requires_grad]
        if optimizer == "sgd":
            if params[0].is_cuda and params[0].dtype in (torch.bfloat16, torch.float16):
                from .ops.optim import FusedSGD
                self.opt = FusedSGD(params, lr=lr)
            else:
                self.opt = torch.optim.SGD(params, lr=lr, foreach=True)
        elif optimizer == "adamw":
            self.opt = torch.optim.AdamW(params, lr=lr, fused=params[0].is_cuda)
        else:
            raise ValueError(optimizer)
        self.device = params[0].device
        self.fuse_expert_sgd = bool(fuse_expert_sgd)
        if self.fuse_expert_sgd and (optimizer != "sgd" or expert_dp_group is not None or mean_expert_grads):
            raise ValueError("fuse_expert_sgd needs plain SGD and expert gradients that nothing else uses")
        self.aux_loss = aux_loss
        self._ids = self._labels = None

    def step_device(self, ids: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        """One optimisation step on device tensors; returns the loss tensor (no host sync)."""
        self.opt.zero_grad(set_to_none=True)
        if self.fuse_expert_sgd:
            group = self.opt.param_groups[0]
            for m in self.raw_model.modules():
                if hasattr(m, "fuse_sgd") and hasattr(m, "experts"):
                    m.fuse_sgd(group["lr"], group.get("weight_decay", 0.0))
        loss = self.model(ids, labels)
        if self.aux_loss:
            aux = self.raw_model.aux_loss()
            if aux is not None:
                loss = loss + aux.to(loss.dtype).sum()
        loss.backward()
        if self.distributed and not self.use_ddp:
            allreduce_replicated_grads(self.raw_model, self.dp_group)
        if self.expert_dp_group is not None or self.mean_expert_grads:
            scale = 1.0 / dist.get_world_size(self.dp_group) if (self.mean_expert_grads and dist.is_initialized()) else None
            reduce_expert_grads(self.raw_model, self.expert_dp_group, scale)
        self.opt.step()
        return loss.detach()

    def step(self, ids: torch.Tensor, labels: Optional[torch.Tensor] = None) -> float:
        """ids/labels: host tensors (pinned for an asynchronous copy). Returns the loss."""
        if labels is None:
            labels = ids
        if self._ids is None or self._ids.shape != ids.shape:
            self._ids = torch.empty(ids.shape, dtype=ids.dtype, device=self.device)
            self._labels = torch.empty(labels.shape, dtype=labels.dtype, device=self.device)
        self._ids.copy_(ids, non_blocking=True)
        self._labels.copy_(labels, non_blocking=True)
        return float(self.step_device(self._ids, self._labels).item())
