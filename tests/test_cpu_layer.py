"""CPU plumbing: the gloo all-to-all path against the dense oracle (fwd and grads)."""
import torch
import pytest

from ccfuser_b200 import MoEConfig, MoELayer, MixMOETransformerMLP
from ccfuser_b200.ops.reference import dense_moe_oracle
from tests.mp_util import run_ranks


def _full_params(cfg, seed, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    e, d, f = cfg.num_experts, cfg.d_model, cfg.d_ffn
    p = {
        "gate.weight": torch.randn(e, d, generator=g) * 0.02,
        "gate.bias": torch.randn(e, generator=g) * 0.02,
        "htoh4.weight": torch.randn(e, f, d, generator=g) * 0.02,
        "htoh4.bias": torch.randn(e, f, generator=g) * 0.02,
        "h4toh.weight": torch.randn(e, d, f, generator=g) * 0.02,
        "h4toh.bias": torch.randn(e, d, generator=g) * 0.02,
    }
    if cfg.activation == "swiglu":
        p["htoh4_gate.weight"] = torch.randn(e, f, d, generator=g) * 0.02
        p["htoh4_gate.bias"] = torch.randn(e, f, generator=g) * 0.02
    return {k: v.to(dtype) for k, v in p.items()}


def load_shard(layer, full, rank):
    e_loc = layer.config.experts_per_rank
    sl = slice(rank * e_loc, (rank + 1) * e_loc)
    with torch.no_grad():
        layer.gate.gate.weight.copy_(full["gate.weight"])
        layer.gate.gate.bias.copy_(full["gate.bias"])
        for name in ("htoh4", "h4toh", "htoh4_gate"):
            if name + ".weight" in full and hasattr(layer.experts, name):
                getattr(layer.experts, name).weight.copy_(full[name + ".weight"][sl])
                getattr(layer.experts, name).bias.copy_(full[name + ".bias"][sl])


def _inputs(world, tokens, d, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(tokens, d, generator=g) for _ in range(world)]


def _rank_fn(rank, world, cfg_kw, tokens):
    cfg = MoEConfig(**cfg_kw)
    full = _full_params(cfg, 0)
    layer = MoELayer(cfg)
    load_shard(layer, full, rank)
    x = _inputs(world, tokens, cfg.d_model)[rank].clone().requires_grad_(True)
    y = layer(x)
    (y * torch.linspace(-1, 1, y.numel()).view_as(y)).sum().backward()
    grads = {n: p.grad.clone() for n, p in layer.named_parameters()}
    return y.detach(), x.grad.clone(), grads


def _oracle(cfg, world, tokens):
    full = {k: v.clone().requires_grad_(True) for k, v in _full_params(cfg, 0).items()}
    xs = [x.clone().requires_grad_(True) for x in _inputs(world, tokens, cfg.d_model)]
    ys = dense_moe_oracle(xs, full, top_k=cfg.top_k, capacity=cfg.capacity(tokens), activation=cfg.activation)
    loss = sum((y * torch.linspace(-1, 1, y.numel()).view_as(y)).sum() for y in ys)
    loss.backward()
    return ys, xs, full


@pytest.mark.parametrize("activation,cf", [("gelu", 1.25), ("swiglu", 1.0), ("relu", None)])
def test_two_rank_layer_matches_oracle(activation, cf):
    """Per rank 512 tokens (4 x 128), d_model 256, 8 experts (4 per rank), FFN 256->1024->256, top-2."""
    world, tokens = 2, 512
    kw = dict(d_model=256, d_ffn=1024, num_experts=8, top_k=2, capacity_factor=cf, activation=activation,
              dtype=torch.float32, ep_size=world, backend="cpu", max_tokens=tokens)
    cfg = MoEConfig(**kw)
    res = run_ranks(_rank_fn, world, kw, tokens)
    ys, xs, full = _oracle(cfg, world, tokens)
    e_loc = cfg.experts_per_rank
    gate_w = sum(r[2]["gate.gate.weight"] for r in res)
    for r in range(world):
        y, gx, grads = res[r]
        assert torch.allclose(y, ys[r].detach(), atol=1e-5, rtol=1e-4)
        assert torch.allclose(gx, xs[r].grad, atol=1e-5, rtol=1e-4)
        sl = slice(r * e_loc, (r + 1) * e_loc)
        for name in ("htoh4", "h4toh") + (("htoh4_gate",) if activation == "swiglu" else ()):
            assert torch.allclose(grads[f"experts.{name}.weight"], full[name + ".weight"].grad[sl], atol=1e-5, rtol=1e-4)
            assert torch.allclose(grads[f"experts.{name}.bias"], full[name + ".bias"].grad[sl], atol=1e-5, rtol=1e-4)
    # the router is replicated: its gradient is the sum over ranks (what DDP's all-reduce produces)
    assert torch.allclose(gate_w, full["gate.weight"].grad, atol=1e-5, rtol=1e-4)


def test_single_process_and_compat_constructor():
    torch.manual_seed(0)
    layer = MixMOETransformerMLP(gate_type={"type": "top", "k": 2},
                                 experts={"count_per_node": 4, "hidden_size_per_expert": 64, "type": "ffn"},
                                 model_dim=32, world_size=1, total_batch_size=64, backend="cpu")
    keys = set(layer.state_dict().keys())
    assert keys == {"gate.gate.weight", "gate.gate.bias", "experts.htoh4.weight", "experts.htoh4.bias",
                    "experts.h4toh.weight", "experts.h4toh.bias"}
    assert layer.experts.htoh4.weight.shape == (4, 64, 32)
    assert layer.experts.h4toh.weight.shape == (4, 32, 64)
    assert all(getattr(p, "skip_allreduce", False) for p in layer.experts.parameters())
    x = torch.randn(2, 8, 32)
    y = layer(x)
    assert y.shape == x.shape
    full = {k.split(".", 1)[1] if k.startswith("experts.") else "gate." + k.split(".")[-1]: v
            for k, v in layer.state_dict().items()}
    ref = dense_moe_oracle([x.reshape(-1, 32)], full, top_k=2, capacity=None)[0]
    assert torch.allclose(y.reshape(-1, 32), ref, atol=1e-5)


def test_compat_constructor_takes_the_reference_experts_dict():
    # the dict exactly as the reference's scripts build it (mix_moe/mix_moe/examples/mix_moe_ddp.py:109,
    # read at mix_moe/mix_moe/transformer.py:449-450), activation module included
    import torch.nn as nn
    layer = MixMOETransformerMLP(gate_type={"type": "top", "k": 2, "capacity_factor": 0.0, "fp32_gate": True},
                                 experts={"type": "ffn", "num_local_expert": 3, "hidden_size": 48,
                                          "activation_fn": nn.ReLU()},
                                 model_dim=32, expert_rank=0, world_size=1, total_batch_size=64, backend="cpu",
                                 capacity_factor=None)
    assert layer.config.experts_per_rank == 3 and layer.config.d_ffn == 48 and layer.config.activation == "relu"
    assert layer.experts.htoh4.weight.shape == (3, 48, 32)
    y = layer(torch.randn(16, 32))
    assert y.shape == (16, 32)
    with pytest.raises(KeyError):
        MixMOETransformerMLP(gate_type={"k": 2}, experts={"type": "ffn"}, model_dim=32, backend="cpu")


def _empty_rank_fn(rank, world):
    cfg = MoEConfig(d_model=32, d_ffn=64, num_experts=4, top_k=2, capacity_factor=None, activation="gelu",
                    dtype=torch.float32, ep_size=world, backend="cpu", max_tokens=64)
    layer = MoELayer(cfg)
    load_shard(layer, _full_params(cfg, 0), rank)
    tokens = 0 if rank == 1 else 48                       # rank 1 has nothing to route in this call
    x = _inputs(world, 48, 32)[rank][:tokens].clone().requires_grad_(True)
    y = layer(x)
    y.sum().backward()
    return y.detach(), x.grad.clone(), layer.experts.htoh4.weight.grad.clone()


def test_a_rank_without_tokens_still_takes_part():
    world = 2
    res = run_ranks(_empty_rank_fn, world)
    cfg = MoEConfig(d_model=32, d_ffn=64, num_experts=4, top_k=2, capacity_factor=None, activation="gelu", dtype=torch.float32)
    full = {k: v.clone().requires_grad_(True) for k, v in _full_params(cfg, 0).items()}
    xs = [_inputs(world, 48, 32)[0].clone().requires_grad_(True), torch.zeros(0, 32, requires_grad=True)]
    ys = dense_moe_oracle(xs, full, top_k=2, capacity=None, activation="gelu")
    sum(y.sum() for y in ys).backward()
    assert res[1][0].shape == (0, 32)
    assert torch.allclose(res[0][0], ys[0].detach(), atol=1e-5, rtol=1e-4)
    assert torch.allclose(res[0][1], xs[0].grad, atol=1e-5, rtol=1e-4)
    for r in range(world):                                # rank 1's experts still served rank 0's tokens
        assert torch.allclose(res[r][2], full["htoh4.weight"].grad[r * 2:(r + 1) * 2], atol=1e-5, rtol=1e-4)


def test_token_mask_skips_padding_tokens():
    """Masked tokens are not routed: zero output rows, no capacity taken, and the real tokens' outputs are what they
    would be if the padding were not in the batch at all."""
    torch.manual_seed(0)
    cfg = MoEConfig(d_model=32, d_ffn=64, num_experts=4, top_k=2, capacity_factor=1.0, activation="gelu",
                    dtype=torch.float32, backend="cpu", max_tokens=64)
    layer = MoELayer(cfg)
    x = torch.randn(2, 20, 32, requires_grad=True)
    mask = torch.ones(2, 20, dtype=torch.bool)
    mask[0, 12:] = False
    mask[1, 17:] = False
    y = layer(x, token_mask=mask)
    assert (y[~mask] == 0).all() and (y[mask].abs().sum(-1) > 0).all()
    y.sum().backward()
    assert (x.grad[~mask] == 0).all()
    # the same real tokens alone, with the capacity that the padded call used (capacity follows the token count)
    real = x.detach()[mask]
    table = layer.count_table()
    assert int(table.sum()) <= int(mask.sum()) * 2
    from ccfuser_b200.gates import topk_softmax_reference
    idx, score = topk_softmax_reference(layer.gate.logits(real), 2)
    from ccfuser_b200.parallel.a2a import moe_forward_a2a
    want = moe_forward_a2a(real, idx, score, layer.experts, num_experts=4, capacity=cfg.capacity(40), group=None)
    assert torch.allclose(y.detach()[mask], want, atol=1e-6)


def test_shared_ffn_is_added_for_every_token_and_is_replicated():
    torch.manual_seed(0)
    cfg = MoEConfig(d_model=16, d_ffn=32, num_experts=4, top_k=2, activation="swiglu", dtype=torch.float32, backend="cpu",
                    shared_ffn=24)
    layer = MoELayer(cfg)
    plain = MoELayer(cfg.replace(shared_ffn=0))
    plain.load_state_dict({k: v for k, v in layer.state_dict().items() if not k.startswith("shared.")})
    x = torch.randn(9, 16)
    want = plain(x) + layer.shared.expert_forward(0, x)
    assert torch.allclose(layer(x), want, atol=1e-6)
    assert layer.state_dict()["shared.htoh4.weight"].shape == (1, 24, 16)
    # routed experts are tagged for the data-parallel ignore list, the shared FFN is not (it is replicated)
    from ccfuser_b200.parallel.ddp import expert_param_names
    names = expert_param_names(layer)
    assert names and all(n.startswith("experts.") for n in names)
    layer(x).sum().backward()
    assert layer.shared.h4toh.weight.grad is not None


def test_sampled_oracle_check_agrees_and_detects_errors():
    """The sampled fp32 check used at benchmark sizes: zero error for the library path on CPU, and a visible error when
    an output, an input gradient or a weight gradient is off."""
    from ccfuser_b200.ops.reference import sampled_oracle_check
    from ccfuser_b200.parallel.a2a import moe_forward_a2a
    torch.manual_seed(0)
    cfg = MoEConfig(d_model=32, d_ffn=64, num_experts=4, top_k=2, capacity_factor=1.0, activation="swiglu",
                    dtype=torch.float32, backend="cpu", max_tokens=256)
    layer = MoELayer(cfg)
    x = torch.randn(200, 32, requires_grad=True)
    idx, score = layer.gate(x)
    score = score.detach().requires_grad_(True)
    y = moe_forward_a2a(x, idx, score, layer.experts, num_experts=4, capacity=cfg.capacity(200), group=None)
    gy = torch.randn_like(y)
    y.backward(gy)
    res = sampled_oracle_check(layer, x, idx, score, y, gy, x.grad, score.grad, n_sample=50, expert=1)
    assert set(res) >= {"y", "dx", "dscore", "dw1", "dw2", "dwg"} and max(res.values()) < 1e-5
    layer.experts.h4toh.weight.grad[1] *= 1.05
    bad = sampled_oracle_check(layer, x, idx, score, y * 1.02, gy, x.grad * 0.9, score.grad, n_sample=50, expert=1)
    assert bad["y"] > 1e-2 and bad["dx"] > 5e-2 and bad["dw2"] > 2e-2 and bad["dw1"] < 1e-5
