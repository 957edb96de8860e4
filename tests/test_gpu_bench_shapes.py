"""The fused layer at the shapes the benchmarks run (several pair tiles per expert, 64 to 224 k-blocks, 16 to 56 column
tiles), forward and backward on one GPU, checked against an fp32 oracle on a sample: the outputs, input gradients and
gate-weight gradients of 64 tokens, and one expert's weight gradients from all of its rows. The small-shape tests in
test_gpu_fused.py cover every element; these cover the regime the published numbers come from."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,d,f,act,experts,tokens,cf,bias", [
    ("mixtral_like_layer", 4096, 14336, "swiglu", 8, 16384, 1.2, False),
    ("gpt_moe_layer", 2048, 8192, "gelu", 8, 8192, None, True),
])
def test_fused_layer_at_benchmark_shape(name, d, f, act, experts, tokens, cf, bias):
    from ccfuser_b200 import MoEConfig, MoELayer
    from ccfuser_b200.ops.reference import sampled_oracle_check
    torch.manual_seed(0)
    cfg = MoEConfig(d_model=d, d_ffn=f, num_experts=experts, top_k=2, capacity_factor=cf, activation=act, bias=bias,
                    dtype=torch.bfloat16, ep_size=1, backend="fused", max_tokens=tokens)
    layer = MoELayer(cfg, device="cuda")
    with torch.no_grad():
        for p in layer.parameters():
            p.normal_(0, 0.02)
    fm = layer._fused_impl()
    x = torch.randn(tokens, d, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
    idx, w = fm.route(x.detach())
    w = w.detach().requires_grad_(True)
    y = fm.run_experts(x, idx, w)
    gy = torch.randn_like(y)
    y.backward(gy)
    torch.cuda.synchronize()
    layer.check_status()
    # the busiest expert: its capacity clamp (when there is one) is then part of what is checked
    busiest = int(torch.bincount(idx.reshape(-1).long(), minlength=experts).argmax())
    err = sampled_oracle_check(layer, x, idx, w, y, gy, x.grad, w.grad, n_sample=64, expert=busiest)
    assert set(err) >= {"y", "dx", "dscore", "dw1", "dw2"}
    bad = {k: v for k, v in err.items() if not v < 3e-2}
    assert not bad, f"{name}: relative errors above 3e-2: {bad} (all: {err})"
    layer.release()
