"""Fused router kernel (linear + top-k + softmax in one tcgen05 kernel) and its GEMM-free backward against the fp32
reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


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


def test_fused_router_logits_are_differentiable_for_auxiliary_losses():
    """A loss on the fp32 logits (load balance, z-loss) reaches x and the router parameters: dense [T, E] gradient added
    to the selected columns' part, both products on the library's own grouped GEMM."""
    from ccfuser_b200.gates import router_aux_loss
    from ccfuser_b200.ops.gemm import Workspace
    from ccfuser_b200.ops.router import fused_router
    torch.manual_seed(3)
    t, d, e, k = 777, 512, 64, 2
    x = (torch.randn(t, d, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    w = (torch.randn(e, d, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    b = (torch.randn(e, device="cuda") * 0.1).bfloat16().requires_grad_(True)
    idx, wt, logits = fused_router(x, w, b, k, want_logits=True)
    gw = torch.randn_like(wt)
    loss = (wt * gw).sum() + router_aux_loss(logits, idx, e, 0.5, 0.1) * 50
    loss.backward()
    torch.cuda.synchronize()
    Workspace.get(x.device).check("fused router with auxiliary losses")
    xf, wf, bf = (v.detach().float().requires_grad_(True) for v in (x, w, b))
    lg = torch.nn.functional.linear(xf, wf, bf)
    sel = torch.gather(lg, 1, idx.long())
    ((torch.softmax(sel, -1) * gw).sum() + router_aux_loss(lg, idx, e, 0.5, 0.1) * 50).backward()

    def rel(a, r):
        return float((a.float() - r).abs().max() / r.abs().max().clamp_min(1e-6))
    assert rel(x.grad, xf.grad) < 3e-2 and rel(w.grad, wf.grad) < 3e-2 and rel(b.grad, bf.grad) < 3e-2


@pytest.mark.parametrize("fused", [True, False])
def test_nan_logits_keep_expert_ids_in_range(fused):
    """A token whose router logits are NaN (a diverged run) must not produce an expert id outside [0, E): the ids stay
    in range, the row's gate weights are NaN (so the NaN is visible downstream), and the backward pass completes."""
    from ccfuser_b200.ops.fused import topk_softmax
    from ccfuser_b200.ops.router import fused_router
    torch.manual_seed(5)
    t, d, e, k = 256, 256, 16, 2
    x = (torch.randn(t, d, device="cuda") * 0.5).bfloat16()
    x[7] = float("nan")
    x[100, 3] = float("inf")
    x.requires_grad_(True)
    w = (torch.randn(e, d, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    if fused:
        idx, wt = fused_router(x, w, None, k)
    else:
        idx, wt = topk_softmax(torch.nn.functional.linear(x, w), k)
    assert int(idx.min()) >= 0 and int(idx.max()) < e
    assert torch.isnan(wt[7]).all() and not torch.isnan(wt[8]).any()
    assert (idx[7, 0] != idx[7, 1]).item()
    wt.nan_to_num().sum().backward()
    torch.cuda.synchronize()
    assert x.grad is not None and w.grad is not None
