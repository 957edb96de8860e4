"""Routers. Same parameter names as the reference gate (``gate.weight`` / ``gate.bias`` inside the
module, i.e. ``<layer>.gate.gate.weight`` in a state dict; mix_moe/mix_moe/gates/naive_gate.py:22)."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class BaseGate(nn.Module):
    """Holds the expert counts and an auxiliary loss slot (mix_moe/mix_moe/gates/base_gate.py:7-29)."""

    def __init__(self, num_expert: int, world_size: int):
        super().__init__()
        self.world_size = world_size
        self.num_expert = num_expert
        self.tot_expert = world_size * num_expert
        self.loss = None

    def forward(self, x):
        raise NotImplementedError("Base gate cannot be used directly")

    def set_loss(self, loss):
        self.loss = loss

    def get_loss(self, clear: bool = True):
        loss = self.loss
        if clear:
            self.loss = None
        return loss

    @property
    def has_loss(self):
        return self.loss is not None


def topk_softmax_reference(logits: torch.Tensor, k: int):
    """fp32 top-k then softmax over the k selected logits (mix_moe/mix_moe/gates/naive_gate.py:31-38).

    Ties are broken towards the lower expert id so CPU, GPU and the CUDA kernel agree."""
    lg = logits.float()
    e = lg.shape[-1]
    # stable descending order with lowest index first among equals
    order = torch.sort(lg, dim=-1, descending=True, stable=True).indices[..., :k]
    val = torch.gather(lg, -1, order)
    score = torch.softmax(val, dim=-1)
    return order, score


def router_aux_loss(logits: torch.Tensor, idx: torch.Tensor, num_experts: int, balance_coef: float = 0.0,
                    z_coef: float = 0.0):
    """Auxiliary router losses, or None when both coefficients are zero.

    * load balance: ``balance_coef * E * sum_e (fraction of slots routed to e) * (mean router probability of e)``;
    * z-loss: ``z_coef * mean(logsumexp(logits)^2)``, which keeps the logits from drifting to large magnitudes.
    Slots whose expert id lies outside [0, num_experts) are not counted. One definition for every backend."""
    if not (balance_coef and balance_coef > 0) and not (z_coef and z_coef > 0):
        return None
    lg = logits.float()
    loss = lg.new_zeros(())
    if balance_coef and balance_coef > 0:
        flat = idx.reshape(-1).long()
        valid = (flat >= 0) & (flat < num_experts)
        frac = torch.zeros(num_experts, device=lg.device, dtype=torch.float32)
        frac.scatter_add_(0, torch.where(valid, flat, torch.zeros_like(flat)), valid.float())
        frac = frac / valid.sum().clamp_min(1)
        loss = loss + balance_coef * num_experts * (frac * torch.softmax(lg, dim=-1).mean(0)).sum()
    if z_coef and z_coef > 0:
        loss = loss + z_coef * torch.logsumexp(lg, dim=-1).square().mean()
    return loss


class NaiveGate(BaseGate):
    """Linear router + top-k + softmax over the selected logits.

    ``forward`` returns ``(idx [T,k] int64, score [T,k] fp32)``. With ``return_all_scores`` the raw
    logits are returned as a third value. An optional load-balance auxiliary loss (the reference
    sets a dummy zero, naive_gate.py:41) is stored with ``set_loss``.
    """

    def __init__(self, d_model: int, num_expert: int, world_size: int, top_k: int = 2,
                 bias: bool = True, aux_loss_coef: float = 0.0, z_loss_coef: float = 0.0):
        super().__init__(num_expert, world_size)
        self.gate = nn.Linear(d_model, self.tot_expert, bias=bias)
        self.top_k = top_k
        self.aux_loss_coef = aux_loss_coef
        self.z_loss_coef = z_loss_coef

    def logits(self, x: torch.Tensor) -> torch.Tensor:
        """Router logits in the router's own dtype (the input is cast when the router is kept in fp32)."""
        return F.linear(x.to(self.gate.weight.dtype), self.gate.weight, self.gate.bias)

    def forward(self, x: torch.Tensor, return_all_scores: bool = False):
        logits = self.logits(x)
        idx, score = topk_softmax_reference(logits, self.top_k)
        loss = router_aux_loss(logits, idx, self.tot_expert, self.aux_loss_coef, self.z_loss_coef)
        self.set_loss(loss if loss is not None else torch.zeros(1, device=x.device, dtype=torch.float32))
        if return_all_scores:
            return idx, score, logits
        return idx, score


def zipf_router_bias(num_experts: int, s: float = 1.2, scale: float = 1.0, seed: int = 0) -> torch.Tensor:
    """Bias that makes expert popularity follow Zipf(s) when the logits are otherwise exchangeable:
    bias_e = scale * log(p_e) with p_e ~ rank^-s, experts permuted by a fixed seed."""
    ranks = torch.arange(1, num_experts + 1, dtype=torch.float64)
    p = ranks.pow(-s)
    p = p / p.sum()
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(num_experts, generator=g)
    bias = torch.empty(num_experts, dtype=torch.float64)
    bias[perm] = scale * torch.log(p)
    return bias.float()
