"""LayerNorm kernels (csrc/norm.cu) and the grouped column-sum kernel against fp32 references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, r):
    return float((a.float() - r.float()).abs().max() / r.float().abs().max().clamp_min(1e-6))


@pytest.mark.parametrize("rows,d,dtype,bias", [(8192, 2048, torch.bfloat16, True), (1000, 768, torch.float16, True),
                                              (333, 512, torch.bfloat16, False), (7, 1024, torch.bfloat16, True),
                                              (4100, 264, torch.float16, True)])
def test_layernorm_forward_backward(rows, d, dtype, bias):
    from ccfuser_b200.ops.norm import LayerNorm
    torch.manual_seed(rows + d)
    ln = LayerNorm(d, device="cuda", dtype=dtype, bias=bias)
    with torch.no_grad():
        ln.weight.copy_(1 + 0.2 * torch.randn(d, device="cuda"))
        if bias:
            ln.bias.copy_(0.1 * torch.randn(d, device="cuda"))
    x = (torch.randn(rows, d, device="cuda") * 2 + 0.5).to(dtype).requires_grad_(True)
    y = ln(x.view(1, rows, d)).view(rows, d)
    gy = torch.randn_like(y)
    y.backward(gy)
    xf = x.detach().float().requires_grad_(True)
    wf = ln.weight.detach().float().requires_grad_(True)
    bf = ln.bias.detach().float().requires_grad_(True) if bias else None
    yr = torch.nn.functional.layer_norm(xf, (d,), wf, bf, ln.eps)
    yr.backward(gy.float())
    assert _rel(y, yr) < 1e-2
    assert _rel(x.grad, xf.grad) < 2e-2
    assert _rel(ln.weight.grad, wf.grad) < 2e-2
    if bias:
        assert _rel(ln.bias.grad, bf.grad) < 2e-2


def test_layernorm_falls_back_outside_the_kernels_range():
    from ccfuser_b200.ops.norm import LayerNorm
    ln = LayerNorm(4096, device="cuda", dtype=torch.bfloat16)      # beyond 2048: torch path
    x = torch.randn(16, 4096, device="cuda", dtype=torch.bfloat16)
    assert torch.equal(ln(x), torch.nn.functional.layer_norm(x, (4096,), ln.weight, ln.bias, ln.eps))


@pytest.mark.parametrize("rows,n,groups,fp16", [([300, 0, 1025, 64], 1024, 4, False), ([5000], 8192, 1, True),
                                               ([17, 33], 264, 2, False)])
def test_colsum_grouped(rows, n, groups, fp16):
    from ccfuser_b200 import native as N
    dtype = torch.float16 if fp16 else torch.bfloat16
    base, acc = [], 0
    for r in rows:
        base.append(acc)
        acc += (r + 127) // 128 * 128
    x = torch.randn(max(acc, 128), n, device="cuda").to(dtype)
    gb = torch.tensor(base, dtype=torch.int32, device="cuda")
    gr = torch.tensor(rows, dtype=torch.int32, device="cuda")
    out = torch.empty(groups, n, dtype=dtype, device="cuda")
    N.check(N.load().ccf_colsum_grouped(x.data_ptr(), n, n, groups, gb.data_ptr(), gr.data_ptr(), out.data_ptr(), int(fp16),
                                        N.stream_ptr()), "ccf_colsum_grouped")
    ref = torch.stack([x[b:b + r].float().sum(0) for b, r in zip(base, rows)])
    assert torch.allclose(out.float(), ref, atol=0.15, rtol=2e-2)
