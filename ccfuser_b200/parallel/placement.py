"""Expert placement: plan which rank hosts which expert from observed routing counts, and move the experts there
while training runs.

The reference carries this as an unfinished prototype: ``balance_compute`` (mix_moe/mix_moe/layers.py:85-246) and
``get_balanced_assignment`` (mix_moe/mix_moe/transformer.py:257-363) walk a nested GPU-topology list and hand every
expert to the partition that sends it the most tokens, and ``_expert_rebalance``
(mix_moe/csrc/cuda/global_exchange.h:49-101, global_exchange.cpp:65-136) ships whole expert blobs with NCCL
send/recv; the Python call site is commented out (layers.py:216-218) and the router is never told about the move.

Here a placement is realised as a *physical permutation of the model*: expert weights (and their optimizer state)
move between ranks, and the rows of the router's linear layer are permuted the same way. The permuted model computes
the same function (expert identity is only a row index of the router), so the kernels, the routing plan and the
checkpoint layout (rank r owns experts ``[r * E_local, (r + 1) * E_local)``) need no indirection table.

Planning is a host-side decision taken rarely (every few hundred steps), from the ``[source rank, expert]`` count
table every rank already holds after a forward call, so every rank derives the same plan without communication.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn


# ---------------------------------------------------------------------------------------------------------------
# cost model
# ---------------------------------------------------------------------------------------------------------------
def _flatten(topo) -> List[int]:
    if isinstance(topo, int):
        return [topo]
    out: List[int] = []
    for t in topo:
        out.extend(_flatten(t))
    return out


def placement_cost(count_table: torch.Tensor, placement: Sequence[int], experts_per_rank: int) -> Dict[str, object]:
    """Load and traffic of a placement. ``count_table[r, e]`` = rows source rank ``r`` routes to expert ``e``
    (expert ids of the *current* layout); ``placement[p]`` = current id of the expert hosted in slot ``p`` (slot p
    lives on rank ``p // experts_per_rank``). Returns rows computed per rank, their maximum, and how many rows stay
    on / leave their source GPU."""
    ct = count_table.to(torch.int64).cpu()
    w, e = ct.shape
    if sorted(placement) != list(range(e)):
        raise ValueError("placement must be a permutation of the expert ids")
    owner = torch.empty(e, dtype=torch.int64)
    owner[torch.tensor(list(placement))] = torch.arange(e) // experts_per_rank
    per_expert = ct.sum(0)
    rank_rows = torch.zeros(w, dtype=torch.int64).index_add(0, owner, per_expert)
    local = int(ct[owner, torch.arange(e)].sum())
    return {"rank_rows": rank_rows.tolist(), "max_rank_rows": int(rank_rows.max()), "local_rows": local,
            "cross_rows": int(per_expert.sum()) - local}


# ---------------------------------------------------------------------------------------------------------------
# planner
# ---------------------------------------------------------------------------------------------------------------
def plan_placement(count_table: torch.Tensor, experts_per_rank: int, topology=None, slack: float = 0.05) -> List[int]:
    """Choose a placement for the observed counts.

    Two goals, in this order: (1) no rank computes much more than the mean (the step time of an expert-parallel
    layer is the time of its busiest rank), (2) among placements that satisfy (1) within ``slack``, experts sit where
    most of their tokens come from, so fewer rows cross NVLink. ``topology`` is a nested list of ranks, e.g.
    ``[[0, 1], [2, 3]]`` for two NVLink-bridged pairs (the shape the reference hard-codes at layers.py:183); experts are
    first split over the outer groups, then inside each group, with the same rule at every level. ``None`` means one
    flat level, which is what an NVSwitch node is. Experts that already sit on the rank they are assigned to keep their
    slot, so a plan that changes little moves little.

    Returns ``placement`` with ``placement[p]`` = current id of the expert that slot ``p`` should host.
    """
    ct = count_table.to(torch.float64).cpu()
    w, e = ct.shape
    e_loc = experts_per_rank
    if e != w * e_loc:
        raise ValueError(f"count table has {e} experts for {w} ranks x {e_loc} experts per rank")
    topo = topology if topology is not None else list(range(w))
    if sorted(_flatten(topo)) != list(range(w)):
        raise ValueError("topology must name every rank exactly once")
    load = ct.sum(0)
    assigned: Dict[int, List[int]] = {}

    def split(node, experts: List[int]):
        ranks = _flatten(node)
        if isinstance(node, int) or len(ranks) == 1:
            assigned[ranks[0]] = experts
            return
        children = list(node)
        child_ranks = [_flatten(c) for c in children]
        room = [len(r) * e_loc for r in child_ranks]
        got: List[List[int]] = [[] for _ in children]
        cur = [0.0] * len(children)
        target = float(load[experts].sum()) / len(ranks)        # mean rows per rank inside this node
        # heaviest experts first: they decide the balance, the light ones fill the gaps
        for ex in sorted(experts, key=lambda i: (-float(load[i]), i)):
            best, best_key = -1, None
            for c in range(len(children)):
                if len(got[c]) >= room[c]:
                    continue
                per_rank = (cur[c] + float(load[ex])) / len(child_ranks[c])
                over = max(0.0, per_rank - target * (1.0 + slack))
                affinity = float(ct[child_ranks[c], ex].sum())
                home = 1 if (ex // e_loc) in child_ranks[c] else 0
                key = (over, -affinity, -home, per_rank, c)
                if best_key is None or key < best_key:
                    best, best_key = c, key
            got[best].append(ex)
            cur[best] += float(load[ex])
        # greedy leftovers: while the busiest child is above the tolerated load, swap one of its experts with a lighter
        # one of another child (or move it into a free slot) if that lowers the larger of the two loads
        sizes = [len(r) for r in child_ranks]
        for _ in range(4 * len(experts)):
            hot = max(range(len(children)), key=lambda c: cur[c] / sizes[c])
            if cur[hot] / sizes[hot] <= target * (1.0 + slack):
                break
            best_gain, best_move = 0.0, None
            for a in got[hot]:
                for c in range(len(children)):
                    if c == hot:
                        continue
                    options = list(got[c]) + ([None] if len(got[c]) < room[c] else [])
                    for b in options:
                        lb = float(load[b]) if b is not None else 0.0
                        la = float(load[a])
                        new_hot = (cur[hot] - la + lb) / sizes[hot]
                        new_c = (cur[c] - lb + la) / sizes[c]
                        gain = cur[hot] / sizes[hot] - max(new_hot, new_c)
                        if gain > best_gain + 1e-9:
                            best_gain, best_move = gain, (a, c, b)
            if best_move is None:
                break
            a, c, b = best_move
            got[hot].remove(a)
            got[c].append(a)
            cur[hot] -= float(load[a])
            cur[c] += float(load[a])
            if b is not None:
                got[c].remove(b)
                got[hot].append(b)
                cur[c] -= float(load[b])
                cur[hot] += float(load[b])
        for c, child in enumerate(children):
            split(child, got[c])

    split(topo, list(range(e)))
    placement = [-1] * e
    for r in range(w):
        mine = assigned[r]
        if len(mine) != e_loc:
            raise AssertionError("planner produced an uneven assignment")
        stay = [ex for ex in mine if ex // e_loc == r]
        come = sorted(ex for ex in mine if ex // e_loc != r)
        for ex in stay:
            placement[ex] = ex
        free = [p for p in range(r * e_loc, (r + 1) * e_loc) if placement[p] < 0]
        for p, ex in zip(free, come):
            placement[p] = ex
    return placement


def compose(first: Sequence[int], second: Sequence[int]) -> List[int]:
    """Placement equivalent to applying ``first`` and then ``second`` (each relative to the layout it starts from)."""
    return [first[q] for q in second]


# ---------------------------------------------------------------------------------------------------------------
# migration
# ---------------------------------------------------------------------------------------------------------------
def _exchange_rows(t: torch.Tensor, placement: Sequence[int], e_loc: int, rank: int, world: int, group) -> torch.Tensor:
    """t: [E_local, ...] rows of this rank's experts in the current layout -> rows of the new layout."""
    if world == 1:
        return t[torch.tensor(list(placement), device=t.device)].clone()
    flat = t.detach().contiguous().view(e_loc, -1)
    row_bytes = flat.shape[1] * flat.element_size()
    raw = flat.view(torch.uint8).view(e_loc, row_bytes)           # byte copy: any dtype crosses any backend
    send_idx: List[int] = []
    send_splits = [0] * world
    recv_slots: List[int] = []
    recv_splits = [0] * world
    # ascending slot order is destination-major order (slot p lives on rank p // e_loc): the order all_to_all_single sends in
    for p, q in enumerate(placement):
        dst, src = p // e_loc, q // e_loc
        if src == rank:
            send_idx.append(q - rank * e_loc)
            send_splits[dst] += 1
        if dst == rank:
            recv_splits[src] += 1
    # all_to_all_single delivers the pieces ordered by source rank; inside one source they keep slot order
    for src in range(world):
        recv_slots.extend(p - rank * e_loc for p, q in enumerate(placement) if p // e_loc == rank and q // e_loc == src)
    send = raw[torch.tensor(send_idx, device=raw.device, dtype=torch.long)] if send_idx else raw[:0]
    recv = torch.empty(e_loc, row_bytes, dtype=torch.uint8, device=raw.device)
    dist.all_to_all_single(recv, send.contiguous(), recv_splits, send_splits, group=group)
    out = torch.empty_like(raw)
    out[torch.tensor(recv_slots, device=raw.device, dtype=torch.long)] = recv
    return out.view(flat.dtype).view(t.shape)


def _state_tensors(optimizer, p: nn.Parameter):
    if optimizer is None:
        return []
    st = optimizer.state.get(p, {})
    return [(k, v) for k, v in st.items() if torch.is_tensor(v) and v.shape == p.shape]


@torch.no_grad()
def rebalance_experts(layer, placement: Sequence[int], optimizer: Optional[torch.optim.Optimizer] = None) -> None:
    """Move the experts of ``layer`` (a ``MoELayer``) to ``placement`` and permute the router rows to match.

    Collective over the layer's expert-parallel group; every rank passes the same placement. Parameters are updated
    in place (their storage, and hence every pointer the kernels hold, stays valid). Per-parameter optimizer state
    with the parameter's shape (momentum, Adam moments) travels with it. Data-parallel replicas of the group must
    apply the same placement.
    """
    cfg = layer.config
    e_loc, world, rank = cfg.experts_per_rank, cfg.ep_size, layer.ep_rank
    e = cfg.num_experts
    placement = [int(q) for q in placement]
    if sorted(placement) != list(range(e)):
        raise ValueError("placement must be a permutation of range(num_experts)")
    if placement == list(range(e)):
        return
    group = layer.ep_group if world > 1 else None
    for p in layer.experts.parameters():
        if p.shape[0] != e_loc:
            raise ValueError("expert parameters must carry the local expert index first")
        tensors = [("param", p.data)] + _state_tensors(optimizer, p)
        for _, t in tensors:
            t.copy_(_exchange_rows(t, placement, e_loc, rank, world, group))
        if p.grad is not None:
            p.grad = None                                           # gradients of the old layout are meaningless now
    gate = layer.gate
    if hasattr(gate, "permute_experts"):
        gate.permute_experts(placement, optimizer)
    else:
        lin = getattr(gate, "gate", None)
        if not isinstance(lin, nn.Linear) or lin.out_features != e:
            raise TypeError("the gate needs a `gate` nn.Linear over all experts or a permute_experts(placement, optimizer) "
                            "method for its rows to follow the experts")
        perm = torch.tensor(placement, device=lin.weight.device, dtype=torch.long)
        for p in (lin.weight, lin.bias):
            if p is None:
                continue
            for _, t in [("param", p.data)] + _state_tensors(optimizer, p):
                t.copy_(t[perm].clone())
            p.grad = None
    history = getattr(layer, "placement_history", None)
    layer.placement_history = compose(history, placement) if history is not None else list(placement)


def main(argv=None):
    """Offline what-if on a saved ``[ranks, experts]`` count table (a ``torch.save``-d integer tensor), the use the
    reference's scratch script makes of its recorded counts (mix_moe/mix_moe/t.py:142-148):

        python -m ccfuser_b200.parallel.placement counts.pt [--topology "[[0,1],[2,3]]"] [--slack 0.05]
    """
    import argparse
    import json
    ap = argparse.ArgumentParser()
    ap.add_argument("counts", help="file with a [ranks, experts] integer tensor")
    ap.add_argument("--topology", default="", help="nested list of ranks as JSON; default flat")
    ap.add_argument("--slack", type=float, default=0.05)
    a = ap.parse_args(argv)
    ct = torch.load(a.counts, map_location="cpu")
    w, e = ct.shape
    e_loc = e // w
    topo = json.loads(a.topology) if a.topology else None
    pl = plan_placement(ct, e_loc, topo, a.slack)
    out = {"ranks": w, "experts": e, "before": placement_cost(ct, list(range(e)), e_loc),
           "after": placement_cost(ct, pl, e_loc), "moved_experts": sum(1 for p, q in enumerate(pl) if p // e_loc != q // e_loc),
           "placement": pl}
    print(json.dumps(out))
    return out


if __name__ == "__main__":
    main()
