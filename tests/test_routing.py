"""Routing invariants of the shared plan definition."""
import torch
import pytest

from ccfuser_b200.ops.routing import route_local, global_plan, positions_in_expert
from ccfuser_b200.gates import topk_softmax_reference, zipf_router_bias, NaiveGate


def _brute_positions(expert):
    seen = {}
    out = []
    for e in expert.tolist():
        out.append(seen.get(e, 0))
        seen[e] = seen.get(e, 0) + 1
    return torch.tensor(out)


@pytest.mark.parametrize("skew", [False, True])
def test_positions_and_capacity(skew):
    g = torch.Generator().manual_seed(3)
    e, t, k = 16, 300, 2
    logits = torch.randn(t, e, generator=g)
    if skew:
        logits = logits + zipf_router_bias(e, 1.2, 2.0)
    idx, score = topk_softmax_reference(logits, k)
    assert torch.allclose(score.sum(-1), torch.ones(t))
    assert (idx[:, 0] != idx[:, 1]).all()
    plan = route_local(idx, e, capacity=40)
    assert torch.equal(plan.pos, _brute_positions(plan.expert))
    assert torch.equal(plan.keep, plan.pos < 40)
    assert torch.equal(plan.count, torch.bincount(plan.expert[plan.keep], minlength=e))
    assert int(plan.count.max()) <= 40
    assert int(plan.raw_count.sum()) == t * k
    # kept slots of one expert occupy positions 0..count-1 exactly once
    for ex in range(e):
        p = plan.pos[(plan.expert == ex) & plan.keep]
        assert torch.equal(torch.sort(p).values, torch.arange(p.numel()))


def test_global_plan_layout():
    g = torch.Generator().manual_seed(0)
    w, e_loc = 4, 3
    table = torch.randint(0, 300, (w, w * e_loc), generator=g)
    table[1, 5] = 0
    table[:, 7] = 0  # an empty expert
    plan = global_plan(table, e_loc, tile=128)
    assert torch.equal(plan.expert_rows, table.sum(0))
    assert (plan.expert_base % 128 == 0).all()
    for o in range(w):
        base = plan.expert_base[o * e_loc:(o + 1) * e_loc]
        rows = plan.expert_rows[o * e_loc:(o + 1) * e_loc]
        assert base[0] == 0
        # experts do not overlap, sources inside an expert tile the range exactly
        for i in range(e_loc - 1):
            assert base[i] + rows[i] <= base[i + 1]
        assert plan.rank_rows[o] >= base[-1] + rows[-1]
    for ex in range(w * e_loc):
        ends = plan.src_offset[:, ex] + table[:, ex]
        assert plan.src_offset[0, ex] == 0
        assert torch.equal(ends[:-1], plan.src_offset[1:, ex])
        assert ends[-1] == plan.expert_rows[ex]


def test_gate_tie_break_and_shapes():
    logits = torch.zeros(5, 8)
    idx, score = topk_softmax_reference(logits, 2)
    assert torch.equal(idx, torch.tensor([[0, 1]] * 5))
    gate = NaiveGate(16, 4, 2, top_k=2)
    i, s = gate(torch.randn(7, 16))
    assert i.shape == (7, 2) and s.shape == (7, 2) and i.dtype == torch.int64
    assert gate.has_loss


def test_router_auxiliary_losses():
    import torch
    from ccfuser_b200.gates import NaiveGate, router_aux_loss
    torch.manual_seed(0)
    gate = NaiveGate(16, 4, 2, top_k=2, aux_loss_coef=0.01, z_loss_coef=0.001)
    x = torch.randn(50, 16)
    idx, score, logits = gate(x, return_all_scores=True)
    loss = gate.get_loss()
    probs = torch.softmax(logits, -1)
    frac = torch.bincount(idx.reshape(-1), minlength=8).float() / idx.numel()
    want = 0.01 * 8 * (frac * probs.mean(0)).sum() + 0.001 * torch.logsumexp(logits, -1).square().mean()
    assert torch.allclose(loss, want, atol=1e-6) and loss.requires_grad
    assert router_aux_loss(logits, idx, 8, 0.0, 0.0) is None
    # unrouted slots are not counted
    idx2 = idx.clone()
    idx2[:10] = -1
    a = router_aux_loss(logits, idx2, 8, 1.0, 0.0)
    frac2 = torch.bincount(idx2.reshape(-1)[idx2.reshape(-1) >= 0], minlength=8).float() / int((idx2 >= 0).sum())
    assert torch.allclose(a, 8 * (frac2 * probs.mean(0)).sum(), atol=1e-6)
    # no coefficients: the gate keeps its zero placeholder (reference behaviour)
    plain = NaiveGate(16, 4, 2)
    plain(x)
    assert float(plain.get_loss()) == 0.0
