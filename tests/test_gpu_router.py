"""Fused router kernel (linear + top-k + softmax in one tcgen05 kernel) against the fp32 reference.

Opt-in: set CCFUSER_TEST_FUSED_ROUTER=1. The kernel is selected in the layer only with CCFUSER_FUSED_ROUTER=1 and is
kept out of the default GPU suite until it has been through a first supervised run on hardware."""
import os

import pytest
import torch

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(os.environ.get("CCFUSER_TEST_FUSED_ROUTER") != "1",
                                 reason="opt-in: CCFUSER_TEST_FUSED_ROUTER=1")]


@pytest.mark.parametrize("t,d,e,k,dtype,bias", [(128, 64, 8, 2, torch.bfloat16, True),
                                               (1000, 256, 64, 2, torch.bfloat16, True),
                                               (4096, 2048, 64, 2, torch.bfloat16, False),
                                               (777, 1024, 200, 8, torch.float16, True),
                                               (333, 512, 256, 4, torch.bfloat16, True),
                                               (64, 4096, 8, 1, torch.float16, False)])
def test_fused_router_matches_reference(t, d, e, k, dtype, bias):
    from ccfuser_b200.gates import topk_softmax_reference
    from ccfuser_b200.ops.gemm import Workspace
    from ccfuser_b200.ops.router import fused_router
    torch.manual_seed(t + e)
    x = (torch.randn(t, d, device="cuda") * 0.5).to(dtype).requires_grad_(True)
    w = (torch.randn(e, d, device="cuda") * 0.05).to(dtype).requires_grad_(True)
    b = (torch.randn(e, device="cuda") * 0.1).to(dtype).requires_grad_(True) if bias else None
    idx, wt, logits = fused_router(x, w, b, k, want_logits=True)
    torch.cuda.synchronize()
    Workspace.get(x.device).check("fused router")
    ref_logits = torch.nn.functional.linear(x.detach().float(), w.detach().float(), None if b is None else b.detach().float())
    assert torch.allclose(logits, ref_logits, atol=2e-3, rtol=1e-3)
    # selection and weights must be exactly those of the reference applied to the kernel's own logits
    ridx, rw = topk_softmax_reference(logits, k)
    assert torch.equal(idx.long(), ridx)
    assert torch.allclose(wt, rw, atol=1e-6)
    # gradients against autograd through the reference with the same selection
    gw = torch.randn_like(wt)
    (wt * gw).sum().backward()
    xf = x.detach().float().requires_grad_(True)
    wf = w.detach().float().requires_grad_(True)
    bf = None if b is None else b.detach().float().requires_grad_(True)
    lg = torch.nn.functional.linear(xf, wf, bf)
    sel = torch.gather(lg, 1, idx.long())
    (torch.softmax(sel, -1) * gw).sum().backward()

    def rel(a, r):
        return float((a.float() - r).abs().max() / r.abs().max().clamp_min(1e-6))
    assert rel(x.grad, xf.grad) < 3e-2 and rel(w.grad, wf.grad) < 3e-2
    if b is not None:
        assert rel(b.grad, bf.grad) < 3e-2
