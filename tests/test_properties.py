"""Property tests (hypothesis) of the routing rule and of the single-process layer against the dense oracle."""
import pytest
import torch

pytest.importorskip("hypothesis")
from hypothesis import given, settings, strategies as st  # noqa: E402

from ccfuser_b200 import MoEConfig, MoELayer
from ccfuser_b200.ops.reference import dense_moe_oracle
from ccfuser_b200.ops.routing import global_plan, route_local


@settings(max_examples=40, deadline=None)
@given(st.integers(1, 40), st.integers(1, 4), st.integers(1, 12), st.integers(1, 30), st.integers(0, 2 ** 31 - 1),
       st.floats(0.0, 0.5))
def test_routing_rule_invariants(tokens, k, experts, capacity, seed, drop_frac):
    g = torch.Generator().manual_seed(seed)
    idx = torch.randint(0, experts, (tokens, k), generator=g)
    idx[torch.rand(tokens, k, generator=g) < drop_frac] = -1          # slots that are not routed at all
    plan = route_local(idx, experts, capacity)
    flat = idx.reshape(-1)
    assert plan.raw_count.sum() == (flat >= 0).sum()
    assert torch.equal(plan.count, plan.raw_count.clamp(max=capacity)) and plan.keep.sum() == plan.count.sum()
    assert not plan.keep[flat < 0].any()
    for e in range(experts):
        mine = (flat == e).nonzero().view(-1)
        # positions inside an expert follow slot order; exactly the first `capacity` are kept
        assert plan.pos[mine].tolist() == list(range(mine.numel()))
        assert plan.keep[mine].tolist() == [p < capacity for p in range(mine.numel())]


@settings(max_examples=25, deadline=None)
@given(st.integers(1, 4), st.integers(1, 6), st.integers(0, 2 ** 31 - 1))
def test_global_plan_segments_tile_aligned_and_disjoint(world, e_loc, seed):
    g = torch.Generator().manual_seed(seed)
    table = torch.randint(0, 300, (world, world * e_loc), generator=g)
    table[torch.rand(table.shape, generator=g) < 0.3] = 0
    gp = global_plan(table, e_loc)
    assert (gp.expert_base % 128 == 0).all()
    for owner in range(world):
        spans = sorted((int(gp.expert_base[e] + gp.src_offset[r, e]), int(gp.expert_base[e] + gp.src_offset[r, e] + table[r, e]))
                       for e in range(owner * e_loc, (owner + 1) * e_loc) for r in range(world) if table[r, e])
        assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))
        assert not spans or spans[-1][1] <= int(gp.rank_rows[owner])


@settings(max_examples=12, deadline=None)
@given(st.integers(1, 33), st.sampled_from(["gelu", "relu", "swiglu"]), st.integers(1, 3), st.sampled_from([None, 0.5, 1.0, 2.0]),
       st.booleans(), st.integers(0, 10 ** 6))
def test_single_process_layer_matches_oracle(tokens, act, k, cf, bias, seed):
    torch.manual_seed(seed)
    cfg = MoEConfig(d_model=16, d_ffn=24, num_experts=5, top_k=k, capacity_factor=cf, activation=act, bias=bias,
                    dtype=torch.float32, backend="cpu", max_tokens=64)
    layer = MoELayer(cfg)
    x = torch.randn(tokens, 16, requires_grad=True)
    y = layer(x)
    y.square().sum().backward()
    full = {"gate.weight": layer.gate.gate.weight.detach(), "gate.bias": layer.gate.gate.bias.detach()}
    for name in ("htoh4", "h4toh", "htoh4_gate"):
        if hasattr(layer.experts, name):
            m = getattr(layer.experts, name)
            full[name + ".weight"] = m.weight.detach().clone().requires_grad_(True)
            full[name + ".bias"] = None if m.bias is None else m.bias.detach().clone().requires_grad_(True)
    xr = x.detach().clone().requires_grad_(True)
    yr = dense_moe_oracle([xr], full, top_k=k, capacity=cfg.capacity(tokens), activation=act)[0]
    yr.square().sum().backward()
    assert torch.allclose(y, yr, atol=1e-5, rtol=1e-4)
    assert torch.allclose(layer.experts.h4toh.weight.grad, full["h4toh.weight"].grad, atol=1e-5, rtol=1e-3)


def test_one_expert_top1_is_a_dense_ffn():
    torch.manual_seed(0)
    cfg = MoEConfig(d_model=16, d_ffn=32, num_experts=1, top_k=1, activation="gelu", dtype=torch.float32, backend="cpu")
    layer = MoELayer(cfg)
    x = torch.randn(3, 7, 16)
    assert torch.allclose(layer(x), layer.experts.expert_forward(0, x.reshape(-1, 16)).reshape(3, 7, 16), atol=1e-6)


@settings(max_examples=30, deadline=None)
@given(st.integers(1, 4), st.integers(1, 5), st.integers(0, 2 ** 31 - 1), st.booleans())
def test_planned_placement_is_a_balanced_permutation(world, e_loc, seed, nested):
    from ccfuser_b200.parallel.placement import placement_cost, plan_placement
    g = torch.Generator().manual_seed(seed)
    e = world * e_loc
    table = (torch.rand(world, e, generator=g).pow(4) * 1000).long()
    topo = None
    if nested and world == 4:
        topo = [[0, 1], [2, 3]]
    pl = plan_placement(table, e_loc, topo)
    assert sorted(pl) == list(range(e))
    assert pl == plan_placement(table.clone(), e_loc, topo)                       # deterministic
    cost = placement_cost(table, pl, e_loc)
    assert sum(cost["rank_rows"]) == int(table.sum()) and cost["local_rows"] + cost["cross_rows"] == int(table.sum())
    # never worse than leaving every expert where it is by more than the heaviest single expert
    ident = placement_cost(table, list(range(e)), e_loc)
    assert cost["max_rank_rows"] <= ident["max_rank_rows"] + int(table.sum(0).max())


@settings(max_examples=60, deadline=None)
@given(st.integers(1, 6), st.integers(0, 2 ** 31 - 1), st.integers(1, 3), st.booleans(), st.booleans())
def test_pair_kernel_tile_order_covers_every_tile_once(groups, seed, n_tiles, gated, swiglu):
    """The CTA-pair kernel's tile sequence, computed on the host by the kernel's own set-up and decode functions: every
    (group, 256-row tile, column tile) exactly once, the tiles made only of locally pushed rows first."""
    import numpy as np
    from ccfuser_b200 import native as N
    lib = N.load()
    rnd = np.random.RandomState(seed % (2 ** 31))
    rows = rnd.choice([0, 1, 127, 128, 255, 256, 257, 300, 511, 512, 513, 777, 1024, 1200], size=groups).astype(np.int32)
    base = np.zeros(groups, dtype=np.int32)
    for g in range(1, groups):
        base[g] = base[g - 1] + (rows[g - 1] + 127) // 128 * 128
    lb = np.array([rnd.randint(0, r + 1) for r in rows], dtype=np.int32)
    lr = np.array([rnd.randint(0, r - b + 1) for r, b in zip(rows, lb)], dtype=np.int32)
    if rnd.rand() < 0.3:
        lr = (rows - lb).astype(np.int32)                       # local rows reach the end of the group
    bn = 128 if swiglu else 256
    n = n_tiles * bn
    cap = 4096
    out = np.full(cap * 5, -7, dtype=np.int32)
    total = lib.ccf_debug_pair_tile_order(base.ctypes.data, rows.ctypes.data, lb.ctypes.data, lr.ctypes.data, groups, n, 512,
                                          int(gated), int(swiglu), out.ctypes.data, cap)
    want = sum(int((r + 255) // 256) for r in rows) * n_tiles
    assert total == want
    recs = out[:5 * total].reshape(total, 5)
    seen = set()
    last_phase = 0
    for g, row0, n0, rows_pair, phase in recs.tolist():
        i, rem = divmod(row0 - int(base[g]), 256)
        assert rem == 0 and n0 % bn == 0 and 0 <= n0 < n
        assert rows_pair == min(256, int(rows[g]) - i * 256) > 0
        assert (g, i, n0) not in seen
        seen.add((g, i, n0))
        assert phase >= last_phase                             # all phase-A tiles come first
        last_phase = phase
        if phase == 0:
            assert gated
            le = min(int(rows[g]), int(lb[g]) + int(lr[g]))
            assert i * 256 >= lb[g] and (i * 256 + rows_pair <= le)      # only rows this rank pushed itself
    assert len(seen) == want
    if not gated:
        assert (recs[:, 4] == 1).all() if total else True


@settings(max_examples=15, deadline=None)
@given(st.integers(1, 30), st.integers(1, 3), st.sampled_from([None, 1.0]), st.integers(0, 10 ** 6), st.floats(0.0, 0.6))
def test_unrouted_slots_are_ignored_by_the_layer_and_by_the_oracle_alike(tokens, k, cf, seed, frac):
    """Slots with expert id -1 (how replicated experts leave the expert-parallel path) contribute nothing and take no
    capacity, in the all-to-all backend exactly as in the dense oracle."""
    from ccfuser_b200.experts import Experts
    from ccfuser_b200.parallel.a2a import moe_forward_a2a
    torch.manual_seed(seed)
    e, d, f = 4, 8, 12
    experts = Experts(e, d, f, "gelu", True, dtype=torch.float32)
    x = torch.randn(tokens, d)
    idx = torch.randint(0, e, (tokens, k))
    idx[torch.rand(tokens, k) < frac] = -1
    score = torch.rand(tokens, k)
    cfg = MoEConfig(d_model=d, d_ffn=f, num_experts=e, top_k=k, capacity_factor=cf, dtype=torch.float32)
    cap = cfg.capacity(tokens)
    y = moe_forward_a2a(x, idx, score, experts, num_experts=e, capacity=cap, group=None)
    full = {"gate.weight": torch.zeros(e, d), "htoh4.weight": experts.htoh4.weight.detach(), "htoh4.bias": experts.htoh4.bias.detach(),
            "h4toh.weight": experts.h4toh.weight.detach(), "h4toh.bias": experts.h4toh.bias.detach()}
    yr = dense_moe_oracle([x], full, top_k=k, capacity=cap, activation="gelu", routing=[(idx, score)])[0]
    assert torch.allclose(y, yr, atol=1e-5, rtol=1e-4)
    untouched = (idx < 0).all(1)
    assert (y[untouched] == 0).all()


@settings(max_examples=40, deadline=None)
@given(st.integers(1, 4), st.integers(1, 4), st.integers(0, 2 ** 31 - 1), st.integers(1, 12))
def test_clipped_plan_keeps_sources_and_owners_consistent(world, e_loc, seed, buffer_tiles):
    """With a receive buffer that may be too small, what a source expects back equals what the owner processes for it,
    expert by expert: the property that keeps every wait satisfiable when rows are refused."""
    from ccfuser_b200.ops.routing import clipped_plan, global_plan
    g = torch.Generator().manual_seed(seed)
    table = torch.randint(0, 400, (world, world * e_loc), generator=g)
    table[torch.rand(table.shape, generator=g) < 0.25] = 0
    max_rows = buffer_tiles * 128
    cp = clipped_plan(table, e_loc, max_rows)
    gp = global_plan(table, e_loc)
    # per expert: the owner's GEMM rows are exactly the accepted rows of all sources, and they form a prefix of the segment
    assert torch.equal(cp.accepted.sum(0), cp.group_rows)
    assert (cp.accepted <= table).all() and (cp.group_rows <= gp.expert_rows).all()
    for e in range(world * e_loc):
        seen_partial = False
        for r in range(world):                       # sources in rank order: once one is cut, all later ones get nothing
            if seen_partial:
                assert int(cp.accepted[r, e]) == 0 or int(table[r, e]) == 0 or int(cp.accepted[r, e]) == 0
            if cp.accepted[r, e] < table[r, e]:
                seen_partial = True
        assert int(gp.expert_base[e]) + int(cp.group_rows[e]) <= max(max_rows, int(gp.expert_base[e]))
    # per (source, owner): rows sent == rows the owner accepted from that source
    owner = torch.arange(world * e_loc) // e_loc
    for o in range(world):
        assert torch.equal(cp.sent_rows[:, o], cp.accepted[:, owner == o].sum(1))
    # a buffer that is large enough clips nothing
    big = clipped_plan(table, e_loc, int(gp.rank_rows.max()))
    assert torch.equal(big.accepted, table) and not bool(big.overflow.any())
    assert torch.equal(cp.overflow, gp.rank_rows > max_rows)
