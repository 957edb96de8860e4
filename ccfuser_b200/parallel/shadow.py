"""Shadow (replicated) experts for skewed routing: the most popular experts of a step are computed on every rank for
that rank's own tokens instead of drawing all of their tokens to one owner.

The reference reserves three extra expert slots per rank for this (``popular_expert_num = 3``,
mix_moe/mix_moe/transformer.py:449,453) and picks the global top-3 experts of every step
(``select_popular_expert``, transformer.py:365-374; used at transformer.py:160-171), but the extra slots are
independent parameters: they are never filled from the owner's weights and their gradients are never returned, so
the feature only works as a timing experiment. Here the replicas are real:

* selection: the per-expert slot counts of all ranks are summed (one small all-reduce) and the ``n`` largest win,
  ties towards the lower id, so every rank selects the same experts without a host round trip;
* weights: every rank contributes the selected experts it owns (zeros otherwise) to a sum all-reduce, which is a
  broadcast from each owner that needs no host-side knowledge of who owns what;
* gradients: the all-reduce is an autograd function whose backward is again a sum all-reduce, so the owner's
  parameter receives the sum of the replicas' gradients and the parameters stay single-copy;
* the selected experts' slots are taken out of the expert-parallel path (expert id -1 = not routed) and computed
  locally: on the fused backend by the same tcgen05 grouped GEMM kernels, as a second, single-rank instance of the
  fused path whose "experts" are the replicas (``ShadowFused``: no host synchronisation, no library GEMM); on the other
  backends with library GEMMs (``shadow_forward``). They are not subject to the capacity factor, since they draw on
  no shared buffer.

Cost model: replicating one expert moves its weights once per step (forward) and its gradients once (backward),
``2 x 3 x d_model x d_ffn x 2`` bytes for SwiGLU in bf16, instead of its tokens twice in each direction; it pays
when one expert draws more than about ``1.5 x d_ffn`` tokens per rank, i.e. under heavy skew only. Off by default
(``MoEConfig.shadow_experts = 0``).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops.reference import expert_ffn


class _AllReduceSum(torch.autograd.Function):
    """y = sum over the group of x; dx = sum over the group of dy."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        y = x.contiguous().clone()
        if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        if ctx.group is not None and dist.is_initialized() and dist.get_world_size(ctx.group) > 1:
            dist.all_reduce(g, group=ctx.group)
        return g, None


def all_reduce_sum(x: torch.Tensor, group) -> torch.Tensor:
    return _AllReduceSum.apply(x, group)


def select_popular(topk_idx: torch.Tensor, num_experts: int, n: int, group) -> torch.Tensor:
    """Ids [n] (int64, ascending popularity order is not guaranteed, the set is what matters) of the ``n`` experts
    that received the most slots over all ranks in this step. Same result on every rank, no host synchronisation."""
    flat = topk_idx.reshape(-1).to(torch.int64)
    valid = (flat >= 0) & (flat < num_experts)
    counts = torch.zeros(num_experts + 1, dtype=torch.float32, device=flat.device)
    counts.scatter_add_(0, torch.where(valid, flat, torch.full_like(flat, num_experts)),
                        torch.ones(flat.numel(), dtype=torch.float32, device=flat.device))
    counts = counts[:num_experts].contiguous()
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(counts, group=group)
    # stable descending sort: equal counts resolve to the lower expert id on every rank
    order = torch.sort(counts, descending=True, stable=True).indices
    return order[:n]


def gather_shadow_params(experts, shadow_ids: torch.Tensor, rank: int, group) -> Dict[str, Optional[torch.Tensor]]:
    """Stacked parameters ``[n, ...]`` of the selected experts, identical on every rank and differentiable: the
    gradient of a replica flows back to the owner's parameter through the all-reduce."""
    e_loc = experts.htoh4.num_expert
    local = shadow_ids - rank * e_loc
    mine = (local >= 0) & (local < e_loc)
    pick = local.clamp(0, e_loc - 1)
    out: Dict[str, Optional[torch.Tensor]] = {}
    for name in ("htoh4", "htoh4_gate", "h4toh"):
        lin = getattr(experts, name, None)
        for part in ("weight", "bias"):
            p = getattr(lin, part, None) if lin is not None else None
            if p is None:
                out[f"{name}.{part}"] = None
                continue
            sel = p[pick]
            mask = mine.view(-1, *([1] * (sel.dim() - 1))).to(sel.dtype)
            out[f"{name}.{part}"] = all_reduce_sum(sel * mask, group)
    return out


def split_shadow_slots(topk_idx: torch.Tensor, shadow_ids: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (idx for the expert-parallel path with the shadowed slots set to -1, shadow index [T, k] in 0..n-1 or -1)."""
    hit = topk_idx.unsqueeze(-1) == shadow_ids.to(topk_idx.dtype).view(1, 1, -1)          # [T, k, n]
    is_shadow = hit.any(-1)
    which = torch.where(is_shadow, hit.to(torch.int64).argmax(-1), torch.full_like(is_shadow, -1, dtype=torch.int64))
    main_idx = torch.where(is_shadow, torch.full_like(topk_idx, -1), topk_idx)
    return main_idx, which


def shadow_forward(x: torch.Tensor, which: torch.Tensor, score: torch.Tensor, params: Dict[str, Optional[torch.Tensor]],
                   activation: str) -> torch.Tensor:
    """Sum over this rank's shadowed slots of score * FFN_replica(x). x [T, d]; which, score [T, k]."""
    n = params["htoh4.weight"].shape[0]
    d_out = params["h4toh.weight"].shape[1]
    y = torch.zeros(x.shape[0], d_out, dtype=x.dtype, device=x.device)
    for j in range(n):
        tok, slot = (which == j).nonzero(as_tuple=True)
        # a replica without tokens still runs (on zero rows): every rank then builds the same graph and so issues the
        # gradient all-reduces of the backward pass in the same order
        opt = lambda key: None if params[key] is None else params[key][j]  # noqa: E731
        o = expert_ffn(x[tok], params["htoh4.weight"][j], opt("htoh4.bias"), params["h4toh.weight"][j], opt("h4toh.bias"),
                       activation, opt("htoh4_gate.weight") if activation == "swiglu" else None,
                       opt("htoh4_gate.bias") if activation == "swiglu" else None)
        y = y.index_add(0, tok, o * score[tok, slot].to(o.dtype).unsqueeze(1))
    return y


class _ReplicaLayerView:
    """What the fused path reads from a layer, for the replicas: a single-rank configuration with one expert per replica
    and a receive buffer that holds every slot of the rank (a replica takes whatever its rank routes to it)."""

    def __init__(self, layer, n: int):
        cfg = layer.config
        import copy
        c = copy.copy(cfg)
        # set field by field: with fewer replicas than top_k the public constructor's "top_k <= num_experts" check does
        # not apply here (k is only the number of slots per token, most of them not shadowed)
        for key, val in dict(num_experts=n, ep_size=1, shadow_experts=0, capacity_factor=None, backend="fused",
                             recv_factor=1.0).items():
            object.__setattr__(c, key, val)
        self.config = c
        self.experts = layer.experts          # only its device is used
        self.gate = None
        self.ep_rank, self.ep_group = 0, None


class ShadowFused:
    """The replicas' FFN on the fused kernels: ``y = sum over this rank's shadowed slots of score * FFN_replica(x)``
    with routing ``which [T, k]`` (replica index, -1 = not shadowed). Differentiable with respect to x, score and the
    gathered replica parameters (whose gradients return to the owners through ``gather_shadow_params``). The kernels
    push the rows into this rank's own buffers (the dispatch role with one rank), so there is no index list built on the
    host and nothing synchronises."""

    def __init__(self, layer, n: int):
        from ..ops.fused import FusedMoE
        self.fm = FusedMoE(_ReplicaLayerView(layer, n))
        self.fm.native_runtime = False        # parameters are fresh tensors every step: launch with the tensors passed in

    def __call__(self, x, which, score, params, activation):
        from ..ops.fused import _FusedMoEFn
        swiglu = activation == "swiglu"
        tensors = (x, score) + tuple(v for v in params.values() if v is not None)
        self.fm._save_pre = torch.is_grad_enabled() and any(t.requires_grad for t in tensors)
        try:
            return _FusedMoEFn.apply(x.contiguous(), score.float(), which.to(torch.int32), params["htoh4.weight"],
                                     params["htoh4.bias"], params["htoh4_gate.weight"] if swiglu else None,
                                     params["htoh4_gate.bias"] if swiglu else None, params["h4toh.weight"],
                                     params["h4toh.bias"], self.fm)
        finally:
            self.fm._save_pre = True

    def close(self):
        self.fm.close()


def shadow_what_if(count_table: torch.Tensor, n: int, d_model: int, d_ffn: int, activation: str = "gelu",
                   experts_per_rank: Optional[int] = None, elem: int = 2, backward: bool = True) -> Dict[str, float]:
    """Host-side estimate for one step with the ``n`` most popular experts replicated: NVLink bytes per rank that the
    replicas' tokens no longer cost, bytes that moving the replicas' weights (and, in training, their gradients) costs,
    and the load of the busiest rank before and after (rows; a replica's rows are computed where their tokens are).
    ``count_table[r, e]`` = rows rank r routes to expert e."""
    ct = count_table.to(torch.float64).cpu()
    w, e = ct.shape
    e_loc = experts_per_rank or e // w
    load = ct.sum(0)
    ids = torch.sort(load, descending=True, stable=True).indices[:n]
    owner = torch.arange(e) // e_loc
    passes = 2 * (2 if backward else 1)                    # rows go out and come back, in forward and in backward
    saved = 0.0
    for i in ids.tolist():
        remote = ct[:, i].clone()
        remote[owner[i]] = 0.0                             # the owner's own rows never crossed NVLink
        saved += float(remote.sum()) * d_model * elem * passes
    mats = 3 if activation == "swiglu" else 2
    # an all-reduce moves about 2 (W - 1) / W of the buffer per rank; once for the weights, once for their gradients
    added = n * mats * d_model * d_ffn * elem * 2.0 * (w - 1) / w * (2 if backward else 1) * w
    rank_rows = torch.zeros(w, dtype=torch.float64).index_add(0, owner, load)
    keep = torch.ones(e, dtype=torch.bool)
    keep[ids] = False
    after = torch.zeros(w, dtype=torch.float64).index_add(0, owner[keep], load[keep]) + ct[:, ids].sum(1)
    return {"experts": ids.tolist(), "nvlink_bytes_saved": saved, "nvlink_bytes_added": added,
            "max_rank_rows_before": float(rank_rows.max()), "max_rank_rows_after": float(after.max()),
            "mean_rank_rows": float(load.sum() / w)}
