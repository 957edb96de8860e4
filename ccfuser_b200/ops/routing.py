"""Routing plan: which (token, slot) goes to which expert row, and what is dropped.

One definition is shared by every backend and by the dense oracle, so that all of them drop the
same tokens:

* slots are numbered token-major, ``s = t * top_k + j``;
* the position of a slot inside its expert is the number of earlier slots of the same rank that
  chose the same expert (a prefix count, so it is deterministic, unlike the ``atomicSub`` placement
  of the reference at mix_moe/csrc/cuda/local_exchange.cu:6-17);
* a slot is kept iff its position is below the per-(rank, expert) capacity;
* a slot whose expert id is negative is not routed at all (it is dropped and counted nowhere), the ``-1 = dropped``
  convention of mix_moe/csrc/cuda/local_exchange.cu:37-70.

The torch implementation below runs on CPU and GPU; the CUDA kernels in csrc/moe_kernels.cu (route_hist_kernel, route_pos_kernel) compute the
same quantities without a host round trip and are tested bit-exactly against it.
"""
from __future__ import annotations

from typing import NamedTuple

import torch


class LocalRouting(NamedTuple):
    """Routing plan of one rank's slots (see route_local)."""
    expert: torch.Tensor   # [S] int64 expert id of each slot
    pos: torch.Tensor      # [S] int64 position of the slot inside (this rank, expert)
    keep: torch.Tensor     # [S] bool  position < capacity
    count: torch.Tensor    # [E] int64 kept rows per expert (after the capacity clamp)
    raw_count: torch.Tensor  # [E] int64 rows per expert before dropping


def positions_in_expert(expert: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Prefix count of equal expert ids, in slot order. expert: [S] int64 -> [S] int64."""
    s = expert.numel()
    if s == 0:
        return expert.new_zeros(0)
    # stable sort keeps slot order inside one expert
    order = torch.sort(expert, stable=True).indices
    sorted_e = expert[order]
    counts = torch.bincount(sorted_e, minlength=num_experts)
    starts = torch.cumsum(counts, 0) - counts
    rank_sorted = torch.arange(s, device=expert.device) - starts[sorted_e]
    pos = torch.empty_like(expert)
    pos[order] = rank_sorted
    return pos


def route_local(topk_idx: torch.Tensor, num_experts: int, capacity: int) -> LocalRouting:
    """topk_idx: [T, k] integer expert ids (negative = not routed) -> plan of this rank's slots."""
    expert = topk_idx.reshape(-1).to(torch.int64)
    valid = (expert >= 0) & (expert < num_experts)
    # unrouted slots are counted in an extra bin so that they never shift the position of a routed slot
    binned = torch.where(valid, expert, torch.full_like(expert, num_experts))
    pos = positions_in_expert(binned, num_experts + 1)
    keep = valid & (pos < capacity)
    raw = torch.bincount(binned, minlength=num_experts + 1)[:num_experts]
    count = torch.clamp(raw, max=capacity)
    return LocalRouting(expert, pos, keep, count, raw)


class GlobalPlan(NamedTuple):
    """Row layout of every rank's receive buffer, computable by every rank from the count table.

    Rows of expert ``e`` on its owner start at ``expert_base[e]`` (a multiple of ``tile``), rows
    sent by source rank ``r`` start at ``expert_base[e] + src_offset[r, e]``.
    """
    expert_rows: torch.Tensor   # [E] int64 rows received by each expert (all sources)
    expert_base: torch.Tensor   # [E] int64 first row of the expert inside its owner's buffer
    src_offset: torch.Tensor    # [W, E] int64 offset of source r's rows inside expert e
    rank_rows: torch.Tensor     # [W] int64 padded rows in use on each owner rank


def global_plan(count_table: torch.Tensor, experts_per_rank: int, tile: int = 128) -> GlobalPlan:
    """count_table: [W, E] kept rows per (source rank, expert)."""
    w, e = count_table.shape
    ct = count_table.to(torch.int64)
    expert_rows = ct.sum(0)
    src_offset = torch.cumsum(ct, 0) - ct
    padded = (expert_rows + tile - 1) // tile * tile
    padded = padded.view(e // experts_per_rank, experts_per_rank)
    base = torch.cumsum(padded, 1) - padded
    rank_rows = padded.sum(1)
    return GlobalPlan(expert_rows, base.reshape(-1), src_offset, rank_rows)


class ClippedPlan(NamedTuple):
    """The row layout when an owner's receive buffer holds only ``max_rows`` rows (what plan_kernel computes on the
    device): rows beyond the buffer are refused by the dispatch role and left out of every count, on both sides."""
    accepted: torch.Tensor     # [W, E] rows of (source, expert) that fit
    sent_rows: torch.Tensor    # [W, W] rows source r sends to owner o (what r's completion wait expects back)
    group_rows: torch.Tensor   # [E] rows each expert's GEMM processes on its owner
    overflow: torch.Tensor     # [W] bool: owner o would have needed more than max_rows


def clipped_plan(count_table: torch.Tensor, experts_per_rank: int, max_rows: int, tile: int = 128) -> ClippedPlan:
    """count_table: [W, E] kept rows per (source rank, expert) after the capacity clamp."""
    gp = global_plan(count_table, experts_per_rank, tile)
    ct = count_table.to(torch.int64)
    w, e = ct.shape
    first = gp.expert_base.view(1, e) + gp.src_offset                       # first row of (r, e) on the owner
    accepted = torch.minimum(ct, (max_rows - first).clamp_min(0))
    owner = torch.arange(e) // experts_per_rank
    sent = torch.zeros(w, w, dtype=torch.int64).index_add(1, owner, accepted)
    group_rows = torch.minimum(gp.expert_rows, (max_rows - gp.expert_base).clamp_min(0))
    return ClippedPlan(accepted, sent, group_rows, gp.rank_rows > max_rows)
