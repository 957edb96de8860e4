"""CUDA-graph replay of the inference forward against eager calls (one GPU)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("act,tokens", [("swiglu", 128), ("gelu", 500)])
def test_graphed_forward_matches_eager(act, tokens):
    from ccfuser_b200.ops.fused import GraphedForward
    from tests.test_gpu_fused import _make_layer
    cfg, layer = _make_layer(act, None, e=8, d=256, f=512, tokens=512)
    xs = [(torch.randn(tokens, cfg.d_model, device="cuda") * 0.5).to(cfg.dtype) for _ in range(3)]
    with torch.no_grad():
        eager = [layer(x).clone() for x in xs]
    g = GraphedForward(layer, tokens)
    for x, want in zip(xs, eager):
        y = g(x)
        torch.cuda.synchronize()
        assert torch.equal(y, want)
    # eager calls keep working next to the graph (the epoch now lives on the device for both)
    with torch.no_grad():
        assert torch.equal(layer(xs[0]), eager[0])
    assert torch.equal(g(xs[1]), eager[1])
    # fewer tokens than the graph was captured for: the padding is masked out of the routing
    short = xs[2][:tokens // 3]
    with torch.no_grad():
        want = layer(short).clone()
    got = g(short)
    torch.cuda.synchronize()
    assert got.shape == want.shape and torch.equal(got, want)
    layer.check_status()
    layer.release()
