"""Library all-to-all expert parallelism: ``all_to_all_single`` (NCCL on GPU, gloo on CPU) around
per-expert library matmuls. On GPU this is only the *baseline* the fused kernels are measured against
(the role FastMoE's global_scatter/global_gather play for the reference,
mix_moe/csrc/cuda/global_exchange.h:104-195); on CPU it is the plumbing test path.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops.routing import route_local


class _AllToAll(torch.autograd.Function):
    """Uneven all_to_all_single over dim 0 with the transposed exchange as its backward."""

    @staticmethod
    def forward(ctx, x, out_splits: List[int], in_splits: List[int], group):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        if group is None or dist.get_world_size(group) == 1:
            out.copy_(x)
        else:
            dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        gi = g.new_empty((sum(ctx.in_splits),) + tuple(g.shape[1:]))
        if ctx.group is None or dist.get_world_size(ctx.group) == 1:
            gi.copy_(g)
        else:
            dist.all_to_all_single(gi, g.contiguous(), ctx.in_splits, ctx.out_splits, group=ctx.group)
        return gi, None, None, None


def all_to_all(x, out_splits, in_splits, group):
    return _AllToAll.apply(x, out_splits, in_splits, group)


def exchange_counts(count: torch.Tensor, world: int, group) -> torch.Tensor:
    """count [E_total] kept rows of this rank per expert -> table [W, E_total] of every rank's counts
    (the reference's expert_all_gather, mix_moe/csrc/cuda/global_exchange.cpp:139-177)."""
    if world == 1:
        return count.view(1, -1).clone()
    table = torch.empty(world * count.numel(), dtype=count.dtype, device=count.device)
    dist.all_gather_into_tensor(table, count.contiguous().view(-1), group=group)
    return table.view(world, count.numel())


def _use_grouped_mm(rows: torch.Tensor, experts) -> bool:
    return (rows.is_cuda and rows.dtype == torch.bfloat16 and hasattr(torch, "_grouped_mm")
            and rows.shape[1] % 8 == 0 and experts.htoh4.weight.shape[1] % 8 == 0)


def _experts_grouped_mm(rows: torch.Tensor, per_expert: List[int], experts) -> torch.Tensor:
    """All local experts with the library grouped GEMM (one call per projection instead of a loop over experts)."""
    import torch.nn.functional as F
    offs = torch.tensor(per_expert, device=rows.device, dtype=torch.int32).cumsum(0).to(torch.int32)
    eid = torch.repeat_interleave(torch.arange(len(per_expert), device=rows.device),
                                  torch.tensor(per_expert, device=rows.device))

    def proj(x, lin):
        y = torch._grouped_mm(x, lin.weight.transpose(1, 2), offs=offs)
        return y if lin.bias is None else y + lin.bias[eid]

    h = proj(rows, experts.htoh4)
    if experts.activation == "swiglu":
        h = F.silu(proj(rows, experts.htoh4_gate)) * h
    elif experts.activation == "gelu":
        h = F.gelu(h)
    else:
        h = F.relu(h)
    return proj(h, experts.h4toh)


def moe_forward_a2a(x: torch.Tensor, topk_idx: torch.Tensor, topk_score: torch.Tensor, experts,
                    *, num_experts: int, capacity: int, group, grouped_mm: bool = False,
                    stats: Optional[dict] = None) -> torch.Tensor:
    """x [T,d]; topk_idx/topk_score [T,k] (a negative expert id = slot not routed). Differentiable w.r.t. x,
    topk_score and the expert params. ``stats`` (optional dict) receives the ``[rank, expert]`` count table."""
    world = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
    e_loc = num_experts // world
    t, d = x.shape
    k = topk_idx.shape[1]
    plan = route_local(topk_idx, num_experts, capacity)
    kept = plan.keep.nonzero(as_tuple=True)[0]                     # slot ids, ascending
    # order kept slots by (expert, position) == stable sort by expert
    order = kept[torch.sort(plan.expert[kept], stable=True).indices]
    send_rows = x[order // k]                                       # [S_kept, d]
    table = exchange_counts(plan.count, world, group)               # [W, E]
    if stats is not None:
        stats["count_table"] = table
    # rows I send to owner o / rows I receive from source r (per local expert)
    send_per_rank = plan.count.view(world, e_loc).sum(1).tolist()
    me = dist.get_rank(group) if world > 1 else 0
    recv_cnt = table[:, me * e_loc:(me + 1) * e_loc]                # [W, e_loc]
    recv_per_rank = recv_cnt.sum(1).tolist()
    recv = all_to_all(send_rows, recv_per_rank, send_per_rank, group)   # grouped by (src, expert)
    # regroup to expert-major: rows of (src r, expert e) are contiguous in `recv`
    rc = recv_cnt.reshape(-1).tolist()
    pieces = list(torch.split(recv, rc, 0))
    seg_ids = [r * e_loc + e for e in range(e_loc) for r in range(world)]          # expert-major order of segments
    rows = torch.cat([pieces[i] for i in seg_ids], 0) if pieces else recv
    per_expert = [sum(rc[r * e_loc + e] for r in range(world)) for e in range(e_loc)]
    if _use_grouped_mm(rows, experts):
        out = _experts_grouped_mm(rows, per_expert, experts)
    else:
        outs_e = []
        for e, rows_e in enumerate(torch.split(rows, per_expert, 0)):
            outs_e.append(experts.expert_forward(e, rows_e) if rows_e.shape[0]
                          else rows_e.new_zeros(0, experts.h4toh.weight.shape[1]))
        out = torch.cat(outs_e, 0)
    # back to the (src, expert) order of the exchange
    outs: List[Optional[torch.Tensor]] = [None] * len(pieces)
    for i, piece in zip(seg_ids, torch.split(out, [rc[i] for i in seg_ids], 0)):
        outs[i] = piece
    back = torch.cat(outs, 0) if outs else recv.new_zeros(0, d)
    ret = all_to_all(back, send_per_rank, recv_per_rank, group)     # same order as send_rows
    w = topk_score.reshape(-1)[order].to(ret.dtype).unsqueeze(1)
    y = torch.zeros(t, ret.shape[1], dtype=ret.dtype, device=x.device)
    y = y.index_add(0, order // k, ret * w)
    return y
