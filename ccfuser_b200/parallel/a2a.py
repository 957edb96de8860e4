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


def _experts_grouped_mm(rows: torch.Tensor, offs: torch.Tensor, eid: torch.Tensor, experts) -> torch.Tensor:
    """All local experts with the library grouped GEMM (one call per projection instead of a loop over experts).
    ``offs`` [E_loc] int32: end row of each expert inside ``rows``; ``eid`` [R]: local expert of each row (for the
    biases). Both are device tensors: nothing here touches the host."""
    import torch.nn.functional as F

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
    topk_score and the expert params. ``stats`` (optional dict) receives the ``[rank, expert]`` count table.

    Host involvement per call: ONE device-to-host read (the 2 W row counts that ``all_to_all_single`` needs as Python
    integers; a dropless exchange of variable size cannot do with less). Sorting, regrouping to expert-major order and
    its inverse are index gathers computed on the device; on bf16 CUDA tensors the experts run as library grouped GEMMs
    with device-side offsets."""
    world = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
    e_loc = num_experts // world
    t, d = x.shape
    k = topk_idx.shape[1]
    dev = x.device
    plan = route_local(topk_idx, num_experts, capacity)
    table = exchange_counts(plan.count, world, group)               # [W, E]
    if stats is not None:
        stats["count_table"] = table
    me = dist.get_rank(group) if world > 1 else 0
    recv_cnt = table[:, me * e_loc:(me + 1) * e_loc]                # [W, e_loc] rows of (source r, local expert e)
    # the one host read: rows I send to each owner, rows I receive from each source
    sizes = torch.cat([plan.count.view(world, e_loc).sum(1), recv_cnt.sum(1)]).tolist()
    send_per_rank, recv_per_rank = [int(v) for v in sizes[:world]], [int(v) for v in sizes[world:]]
    n_send, n_recv = sum(send_per_rank), sum(recv_per_rank)
    # kept slots ordered by (expert, position): a stable sort by expert with the dropped slots keyed past the end
    key = torch.where(plan.keep, plan.expert, torch.full_like(plan.expert, num_experts))
    order = torch.sort(key, stable=True).indices[:n_send]
    send_rows = x[order // k]                                       # [S_kept, d]
    recv = all_to_all(send_rows, recv_per_rank, send_per_rank, group)   # segments ordered (source, expert)
    # regroup to expert-major: row i of `recv` belongs to segment seg[i] = source * e_loc + expert
    seg_len = recv_cnt.reshape(-1)
    seg = torch.repeat_interleave(torch.arange(world * e_loc, device=dev), seg_len, output_size=n_recv)
    row_expert = seg % e_loc
    perm = torch.sort(row_expert * world + seg // e_loc, stable=True).indices     # expert-major, sources in rank order
    rows = recv[perm]
    per_expert = recv_cnt.sum(0)                                    # [e_loc] device
    if _use_grouped_mm(rows, experts):
        offs = per_expert.cumsum(0).to(torch.int32)
        out = _experts_grouped_mm(rows, offs, row_expert[perm], experts)
    else:
        counts = [int(v) for v in per_expert.tolist()]              # CPU / fp32 plumbing path: a per-expert loop
        outs_e = []
        for e, rows_e in enumerate(torch.split(rows, counts, 0)):
            outs_e.append(experts.expert_forward(e, rows_e) if rows_e.shape[0]
                          else rows_e.new_zeros(0, experts.h4toh.weight.shape[1]))
        out = torch.cat(outs_e, 0) if outs_e else rows.new_zeros(0, experts.h4toh.weight.shape[1])
    # back to the (source, expert) order of the exchange: the inverse gather
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(n_recv, device=dev)
    back = out[inv]
    ret = all_to_all(back, send_per_rank, recv_per_rank, group)     # same order as send_rows
    w = topk_score.reshape(-1)[order].to(ret.dtype).unsqueeze(1)
    y = torch.zeros(t, ret.shape[1], dtype=ret.dtype, device=dev)
    y = y.index_add(0, order // k, ret * w)
    return y
