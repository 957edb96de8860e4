"""Expert placement planner, live expert migration and shadow (replicated) experts, on gloo ranks."""
import torch

from ccfuser_b200 import MoEConfig, MoELayer
from ccfuser_b200.ops.reference import dense_moe_oracle
from ccfuser_b200.ops.routing import route_local
from ccfuser_b200.parallel.placement import compose, placement_cost, plan_placement
from tests.mp_util import run_ranks
from tests.test_cpu_layer import _full_params, _inputs, load_shard


# ---------------------------------------------------------------------------------------------------------------
# planner (pure host code)
# ---------------------------------------------------------------------------------------------------------------
def test_planner_balances_skewed_counts():
    w, e_loc = 4, 4
    g = torch.Generator().manual_seed(0)
    ct = torch.randint(10, 40, (w, w * e_loc), generator=g)
    ct[:, 0:4] += 400                       # all four hot experts start on rank 0
    ident = list(range(w * e_loc))
    before = placement_cost(ct, ident, e_loc)
    pl = plan_placement(ct, e_loc)
    after = placement_cost(ct, pl, e_loc)
    assert sorted(pl) == ident
    assert after["max_rank_rows"] < 0.5 * before["max_rank_rows"]
    # one hot expert per rank is the only balanced answer
    owners = sorted(pl.index(h) // e_loc for h in range(4))
    assert owners == [0, 1, 2, 3]
    # the hot expert that stays on rank 0 keeps its slot
    assert any(pl[h] == h for h in range(4))


def test_planner_prefers_locality_when_balanced():
    w, e_loc = 2, 2
    # every expert has the same load; experts 0,1 get their tokens from rank 1 and experts 2,3 from rank 0
    ct = torch.tensor([[0, 0, 100, 100], [100, 100, 0, 0]])
    pl = plan_placement(ct, e_loc)
    c = placement_cost(ct, pl, e_loc)
    assert c["cross_rows"] == 0 and c["local_rows"] == 400
    assert placement_cost(ct, [0, 1, 2, 3], e_loc)["cross_rows"] == 400


def test_planner_follows_nested_topology():
    w, e_loc = 4, 1
    # expert 0 is fed by ranks 2,3; expert 2 by ranks 0,1; the rest is uniform
    ct = torch.tensor([[0, 10, 50, 10], [0, 10, 50, 10], [50, 10, 0, 10], [50, 10, 0, 10]])
    pl = plan_placement(ct, e_loc, topology=[[0, 1], [2, 3]])
    assert pl.index(0) in (2, 3) and pl.index(2) in (0, 1)
    assert compose([1, 0, 3, 2], [2, 3, 0, 1]) == [3, 2, 1, 0]


def test_route_local_skips_negative_ids():
    idx = torch.tensor([[0, -1], [0, 1], [-1, -1], [0, 1]])
    plan = route_local(idx, 2, capacity=2)
    assert plan.count.tolist() == [2, 2] and plan.raw_count.tolist() == [3, 2]
    assert plan.keep.tolist() == [True, False, True, True, False, False, False, True]
    assert plan.pos[plan.keep].tolist() == [0, 1, 0, 1]


# ---------------------------------------------------------------------------------------------------------------
# live migration
# ---------------------------------------------------------------------------------------------------------------
def _rebalance_fn(rank, world, kw, tokens, placement):
    cfg = MoEConfig(**kw)
    layer = MoELayer(cfg)
    load_shard(layer, _full_params(cfg, 0), rank)
    opt = torch.optim.SGD(layer.parameters(), lr=0.0, momentum=0.9)
    x = _inputs(world, tokens, cfg.d_model)[rank]
    y0 = layer(x)
    y0.square().sum().backward()
    opt.step()                                                  # lr 0: parameters unchanged, momentum buffers = grads
    mom_before = {n: opt.state[p]["momentum_buffer"].clone() for n, p in layer.named_parameters()}
    ptrs = {n: p.data_ptr() for n, p in layer.named_parameters()}
    used = layer.rebalance(placement, optimizer=opt)
    assert all(p.data_ptr() == ptrs[n] for n, p in layer.named_parameters())       # updated in place
    y1 = layer(x)
    planned = layer.rebalance(optimizer=opt)                    # plan from the counts of the call above
    y2 = layer(x)
    mom_after = {n: opt.state[p]["momentum_buffer"].clone() for n, p in layer.named_parameters()}
    sd = {k: v.clone() for k, v in layer.state_dict().items()}
    return y0.detach(), y1.detach(), y2.detach(), mom_before, mom_after, sd, used, planned, layer.placement_history


def test_live_rebalance_keeps_the_function_and_moves_optimizer_state():
    world, tokens = 2, 96
    kw = dict(d_model=32, d_ffn=64, num_experts=8, top_k=2, capacity_factor=None, activation="swiglu",
              dtype=torch.float32, ep_size=world, backend="cpu", max_tokens=tokens)
    placement = [5, 1, 6, 3, 4, 0, 2, 7]                        # experts 0<->5 and 2<->6 change rank
    res = run_ranks(_rebalance_fn, world, kw, tokens, placement)
    cfg = MoEConfig(**kw)
    full = _full_params(cfg, 0)
    e_loc = cfg.experts_per_rank
    for r in range(world):
        y0, y1, y2, mom_b, mom_a, sd, used, planned, hist = res[r]
        assert used == placement
        assert torch.allclose(y0, y1, atol=1e-6) and torch.allclose(y0, y2, atol=1e-6)
        assert sorted(planned) == list(range(8)) and planned == res[0][7]          # same plan on every rank
        assert sorted(hist) == list(range(8)) and hist == res[0][8]
        # after both moves slot p of the model holds original expert hist[p]: weights, router rows
        for p_local in range(e_loc):
            orig = hist[r * e_loc + p_local]
            assert torch.equal(sd["experts.htoh4.weight"][p_local], full["htoh4.weight"][orig])
            assert torch.equal(sd["experts.h4toh.bias"][p_local], full["h4toh.bias"][orig])
        assert torch.equal(sd["gate.gate.weight"], full["gate.weight"][torch.tensor(hist)])
    # momentum buffers travelled with their experts: compare against the pre-move buffers of the rank that owned them
    hist = res[0][8]
    for r in range(world):
        for p_local in range(e_loc):
            orig = hist[r * e_loc + p_local]
            src_rank, src_local = orig // e_loc, orig % e_loc
            for key in ("experts.htoh4.weight", "experts.htoh4_gate.bias", "experts.h4toh.weight"):
                assert torch.equal(res[r][4][key][p_local], res[src_rank][3][key][src_local])
        assert torch.equal(res[r][4]["gate.gate.bias"], res[r][3]["gate.gate.bias"][torch.tensor(hist)])


# ---------------------------------------------------------------------------------------------------------------
# shadow experts
# ---------------------------------------------------------------------------------------------------------------
def _shadow_fn(rank, world, kw, tokens):
    cfg = MoEConfig(**kw)
    full = _full_params(cfg, 0)
    full["gate.bias"][5] += 1.0                                  # make expert 5 (rank 1) clearly the most popular
    layer = MoELayer(cfg)
    load_shard(layer, full, rank)
    x = _inputs(world, tokens, cfg.d_model)[rank].clone().requires_grad_(True)
    y = layer(x)
    (y * torch.linspace(-1, 1, y.numel()).view_as(y)).sum().backward()
    grads = {n: p.grad.clone() for n, p in layer.named_parameters()}
    return y.detach(), x.grad.clone(), grads, layer.last_stats["shadow_ids"], layer.count_table()


def test_shadow_experts_match_the_oracle_and_return_gradients_to_the_owner():
    world, tokens = 2, 128
    kw = dict(d_model=32, d_ffn=64, num_experts=8, top_k=2, capacity_factor=None, activation="gelu",
              dtype=torch.float32, ep_size=world, backend="cpu", max_tokens=tokens, shadow_experts=2)
    cfg = MoEConfig(**kw)
    res = run_ranks(_shadow_fn, world, kw, tokens)
    full = _full_params(cfg, 0)
    full["gate.bias"][5] += 1.0
    full = {k: v.clone().requires_grad_(True) for k, v in full.items()}
    xs = [x.clone().requires_grad_(True) for x in _inputs(world, tokens, cfg.d_model)]
    ys = dense_moe_oracle(xs, full, top_k=cfg.top_k, capacity=None, activation=cfg.activation)
    sum((y * torch.linspace(-1, 1, y.numel()).view_as(y)).sum() for y in ys).backward()
    e_loc = cfg.experts_per_rank
    shadow = res[0][3].tolist()
    assert 5 in shadow and res[1][3].tolist() == shadow
    for r in range(world):
        y, gx, grads, _, table = res[r]
        assert torch.allclose(y, ys[r].detach(), atol=1e-5, rtol=1e-4)
        assert torch.allclose(gx, xs[r].grad, atol=1e-5, rtol=1e-4)
        sl = slice(r * e_loc, (r + 1) * e_loc)
        # owners hold the complete gradient of their experts, shadowed ones included (summed over the replicas)
        for name in ("htoh4", "h4toh"):
            assert torch.allclose(grads[f"experts.{name}.weight"], full[name + ".weight"].grad[sl], atol=1e-5, rtol=1e-4)
            assert torch.allclose(grads[f"experts.{name}.bias"], full[name + ".bias"].grad[sl], atol=1e-5, rtol=1e-4)
        # no row of a shadowed expert went through the exchange
        assert int(table[:, shadow].sum()) == 0
    gate_w = sum(r[2]["gate.gate.weight"] for r in res)
    assert torch.allclose(gate_w, full["gate.weight"].grad, atol=1e-5, rtol=1e-4)


# ---------------------------------------------------------------------------------------------------------------
# re-placement inside a training loop (the sequence bench.py --rebalance runs)
# ---------------------------------------------------------------------------------------------------------------
def _train_rebalance_fn(rank, world):
    from ccfuser_b200.models.gpt_moe import GPTMoE, GPTMoEConfig
    from ccfuser_b200.train import TrainStep
    torch.manual_seed(0)
    c = GPTMoEConfig(vocab_size=128, n_layer=4, n_head=2, d_model=32, d_ffn=64, seq_len=16, num_experts=8, top_k=2,
                     ep_size=world, backend="cpu", max_tokens=64, dtype=torch.float32)
    model = GPTMoE(c)
    trainer = TrainStep(model, lr=1e-2, optimizer="sgd")
    g = torch.Generator().manual_seed(10 + rank)
    ids = torch.randint(0, 128, (4, 16), generator=g)
    labels = ids.roll(-1, 1)
    for _ in range(2):
        trainer.step_device(ids, labels)
    with torch.no_grad():
        before = float(model(ids, labels))
    moved = 0
    for m in model.moe_layers():
        pl = m.rebalance(optimizer=trainer.opt)
        moved += sum(1 for slot, old in enumerate(pl) if slot // 4 != old // 4)
    with torch.no_grad():
        after = float(model(ids, labels))
    l1 = float(trainer.step_device(ids, labels))
    l2 = float(trainer.step_device(ids, labels))
    return before, after, moved, l1, l2


def test_rebalance_between_training_steps_keeps_the_loss():
    res = run_ranks(_train_rebalance_fn, 2)
    for before, after, moved, l1, l2 in res:
        assert abs(before - after) < 1e-5
        assert l2 < l1 + 1e-3                       # training goes on
    assert res[0][2] == res[1][2]
