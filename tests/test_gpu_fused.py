"""Fused layer (one GPU, expert-parallel world of one rank) and its building kernels vs fp32 references."""
import ctypes as C

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def test_topk_softmax_kernel_matches_reference():
    from ccfuser_b200.ops.fused import topk_softmax
    from ccfuser_b200.gates import topk_softmax_reference
    torch.manual_seed(0)
    for e, k, dtype in [(8, 2, torch.bfloat16), (64, 2, torch.bfloat16), (64, 4, torch.float32), (200, 8, torch.float16)]:
        logits = torch.randn(777, e, device="cuda", dtype=dtype)
        logits[5] = 0  # all equal: ties resolve to the lowest ids
        lg = logits.clone().requires_grad_(True)
        idx, w = topk_softmax(lg, k)
        ridx, rw = topk_softmax_reference(logits, k)
        assert torch.equal(idx.long(), ridx)
        assert torch.allclose(w, rw, atol=1e-6)
        gw = torch.randn_like(w)
        (w * gw).sum().backward()
        lf = logits.float().requires_grad_(True)
        _, w2 = topk_softmax_reference(lf, k)
        (w2 * gw).sum().backward()
        assert torch.allclose(lg.grad.float(), lf.grad, atol=2e-2 if dtype != torch.float32 else 1e-5)


@pytest.mark.parametrize("s,e,cap", [(37, 8, 5), (4096, 64, 200), (32768, 64, 1229), (5000, 256, 10000)])
def test_route_kernel_bit_exact(s, e, cap):
    from ccfuser_b200 import native as N
    from ccfuser_b200.ops.routing import route_local
    lib = N.load()
    g = torch.Generator().manual_seed(s)
    p = torch.rand(e, generator=g).pow(3)
    expert = torch.multinomial(p / p.sum(), s, replacement=True, generator=g).int().cuda()
    nb = (s + 1023) // 1024
    pos = torch.empty(s, dtype=torch.int32, device="cuda")
    bh = torch.zeros(nb * e, dtype=torch.int32, device="cuda")
    bo = torch.zeros(nb * e, dtype=torch.int32, device="cuda")
    raw = torch.zeros(e, dtype=torch.int32, device="cuda")
    kept = torch.zeros(e, dtype=torch.int32, device="cuda")
    ticket = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(2):  # second call checks that the ticket returns to zero
        N.check(lib.ccf_route(expert.data_ptr(), s, e, cap, pos.data_ptr(), bh.data_ptr(), bo.data_ptr(),
                              raw.data_ptr(), kept.data_ptr(), ticket.data_ptr(), N.stream_ptr()), "route")
    torch.cuda.synchronize()
    ref = route_local(expert.long().cpu().view(-1, 1), e, cap)
    assert torch.equal(pos.cpu().long(), ref.pos)
    assert torch.equal(raw.cpu().long(), ref.raw_count)
    assert torch.equal(kept.cpu().long(), ref.count)


def test_route_kernel_on_recorded_skew():
    """The recorded 4-rank x 64-expert histogram (a few experts draw thousands of slots, many draw none)."""
    from ccfuser_b200 import native as N
    from ccfuser_b200.ops.routing import route_local
    from tests.fixtures import RECORDED_COUNTS
    lib = N.load()
    e, cap = 64, 512
    i32 = dict(dtype=torch.int32, device="cuda")
    for r, counts in enumerate(RECORDED_COUNTS):
        ids = torch.repeat_interleave(torch.arange(e), torch.tensor(counts))
        ids = ids[torch.randperm(ids.numel(), generator=torch.Generator().manual_seed(r))]
        s = ids.numel()
        expert = ids.int().cuda()
        nb = (s + 1023) // 1024
        pos, bh, bo = torch.empty(s, **i32), torch.zeros(nb * e, **i32), torch.zeros(nb * e, **i32)
        raw, kept, ticket = torch.zeros(e, **i32), torch.zeros(e, **i32), torch.zeros(1, **i32)
        N.check(lib.ccf_route(expert.data_ptr(), s, e, cap, pos.data_ptr(), bh.data_ptr(), bo.data_ptr(),
                              raw.data_ptr(), kept.data_ptr(), ticket.data_ptr(), N.stream_ptr()), "route")
        torch.cuda.synchronize()
        ref = route_local(ids.view(-1, 1), e, cap)
        assert raw.cpu().tolist() == counts
        assert torch.equal(pos.cpu().long(), ref.pos)
        assert torch.equal(kept.cpu().long(), ref.count)


def test_route_ordered_gives_destination_order():
    """ccf_route_ordered: kept slots listed expert by expert starting at `first_expert`, in position order."""
    from ccfuser_b200 import native as N
    lib = N.load()
    s, e, cap, first = 5000, 24, 150, 8
    g = torch.Generator().manual_seed(5)
    expert = torch.randint(0, e, (s,), generator=g).int().cuda()
    nb = (s + 1023) // 1024
    i32 = dict(dtype=torch.int32, device="cuda")
    pos, bh, bo = torch.empty(s, **i32), torch.zeros(nb * e, **i32), torch.zeros(nb * e, **i32)
    raw, kept, ticket = torch.zeros(e, **i32), torch.zeros(e, **i32), torch.zeros(1, **i32)
    order_off, sorted_slot, slot_row = torch.zeros(e + 1, **i32), torch.full((s,), -5, **i32), torch.full((s,), 7, **i32)
    N.check(lib.ccf_route_ordered(expert.data_ptr(), s, e, cap, pos.data_ptr(), bh.data_ptr(), bo.data_ptr(), raw.data_ptr(),
                                  kept.data_ptr(), ticket.data_ptr(), order_off.data_ptr(), sorted_slot.data_ptr(),
                                  slot_row.data_ptr(), first, N.stream_ptr()), "route_ordered")
    torch.cuda.synchronize()
    ex, ps, kp = expert.cpu().long(), pos.cpu().long(), kept.cpu().long()
    order = [(first + k) % e for k in range(e)]
    off, run = {}, 0
    for x in order:
        off[x] = run
        run += int(kp[x])
    assert int(order_off[e]) == run and all(int(order_off[x]) == off[x] for x in range(e))
    ss = sorted_slot.cpu().long()
    for slot in range(s):
        if ps[slot] < cap:
            assert int(ss[off[int(ex[slot])] + int(ps[slot])]) == slot
            assert int(slot_row[slot]) == 7          # left for the dispatch role to fill in
        else:
            assert int(slot_row[slot]) == -1


def _make_layer(act, cf, e=8, d=256, f=512, tokens=1024, k=2, dtype=torch.bfloat16, bias=True):
    from ccfuser_b200 import MoEConfig, MoELayer
    torch.manual_seed(0)
    cfg = MoEConfig(d_model=d, d_ffn=f, num_experts=e, top_k=k, capacity_factor=cf, activation=act, bias=bias,
                    dtype=dtype, ep_size=1, backend="fused", max_tokens=tokens)
    layer = MoELayer(cfg, device="cuda")
    with torch.no_grad():
        for p in layer.parameters():
            p.copy_(torch.randn_like(p) * 0.05)
    return cfg, layer


def _oracle_with_routing(cfg, layer, x, idx, w):
    from ccfuser_b200.ops.reference import dense_moe_oracle
    full = {"gate.weight": layer.gate.gate.weight.detach().float(), "gate.bias": None}
    for name in ("htoh4", "h4toh", "htoh4_gate"):
        if hasattr(layer.experts, name):
            m = getattr(layer.experts, name)
            full[name + ".weight"] = m.weight.detach().float().requires_grad_(True)
            full[name + ".bias"] = None if m.bias is None else m.bias.detach().float().requires_grad_(True)
    xf = x.detach().float().requires_grad_(True)
    wf = w.detach().float().requires_grad_(True)
    y = dense_moe_oracle([xf], full, top_k=cfg.top_k, capacity=cfg.capacity(x.shape[0]),
                         activation=cfg.activation, routing=[(idx, wf)])[0]
    return y, xf, wf, full


def _rel(a, b):
    return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6))


@pytest.mark.parametrize("act,cf,tokens", [("gelu", None, 1024), ("gelu", 1.0, 1000), ("relu", 1.25, 333),
                                            ("swiglu", 1.2, 1024), ("swiglu", None, 77)])
@pytest.mark.parametrize("pair_tiles", [True, False])
def test_fused_layer_forward_backward_one_gpu(act, cf, tokens, pair_tiles, monkeypatch):
    from ccfuser_b200.ops import gemm as G
    from ccfuser_b200.ops.fused import topk_softmax, _FusedMoEFn
    # at these sizes an expert expects fewer rows than one 256-row pair tile, which selects the one-CTA kernel for the
    # row-grouped launches; half of the cases keep the CTA-pair kernel so that both carry the whole layer here
    monkeypatch.setattr(G, "SMALL_ROWS_DEFAULT", 0 if pair_tiles else 320)
    cfg, layer = _make_layer(act, cf, tokens=1024)
    fm = layer._fused_impl()
    x = (torch.randn(tokens, cfg.d_model, device="cuda") * 0.5).to(cfg.dtype).requires_grad_(True)
    # run the expert part with explicit routing so the oracle sees the same decisions
    logits = layer.gate.logits(x.detach())
    idx, w = topk_softmax(logits, cfg.top_k)
    w = w.detach().requires_grad_(True)
    ex = layer.experts
    wg = ex.htoh4_gate.weight if act == "swiglu" else None
    bg = ex.htoh4_gate.bias if act == "swiglu" else None
    y = _FusedMoEFn.apply(x, w, idx, ex.htoh4.weight, ex.htoh4.bias, wg, bg, ex.h4toh.weight, ex.h4toh.bias, fm)
    gy = torch.randn_like(y)
    y.backward(gy)
    torch.cuda.synchronize()
    fm.ctx.check_status("fused test")
    yr, xf, wf, full = _oracle_with_routing(cfg, layer, x, idx, w)
    yr.backward(gy.float())
    assert _rel(y, yr) < 3e-2
    assert _rel(x.grad, xf.grad) < 4e-2
    assert _rel(w.grad, wf.grad) < 4e-2
    assert _rel(ex.htoh4.weight.grad, full["htoh4.weight"].grad) < 4e-2
    assert _rel(ex.htoh4.bias.grad, full["htoh4.bias"].grad) < 4e-2
    assert _rel(ex.h4toh.weight.grad, full["h4toh.weight"].grad) < 4e-2
    assert _rel(ex.h4toh.bias.grad, full["h4toh.bias"].grad) < 4e-2
    if act == "swiglu":
        assert _rel(ex.htoh4_gate.weight.grad, full["htoh4_gate.weight"].grad) < 4e-2
        assert _rel(ex.htoh4_gate.bias.grad, full["htoh4_gate.bias"].grad) < 4e-2
    # dropped slots: no gradient to their gate weight
    from ccfuser_b200.ops.routing import route_local
    plan = route_local(idx.long().cpu(), cfg.num_experts, cfg.capacity(tokens))
    assert (w.grad.cpu().view(-1)[~plan.keep] == 0).all()


def test_fused_layer_fp16_forward_only_one_expert_per_rank():
    """fp16, a single local expert, SwiGLU without biases, forward only (the small-message serving shape)."""
    from ccfuser_b200.ops.fused import topk_softmax, _FusedMoEFn
    for tokens in (128, 500):
        cfg, layer = _make_layer("swiglu", None, e=1, d=256, f=512, tokens=512, k=1, dtype=torch.float16, bias=False)
        fm = layer._fused_impl()
        x = (torch.randn(tokens, 256, device="cuda") * 0.5).half()
        with torch.no_grad():
            idx, w = topk_softmax(layer.gate.logits(x), 1)
            ex = layer.experts
            y = _FusedMoEFn.apply(x, w, idx, ex.htoh4.weight, None, ex.htoh4_gate.weight, None, ex.h4toh.weight, None, fm)
        torch.cuda.synchronize()
        fm.ctx.check_status("fp16 forward")
        yr, *_ = _oracle_with_routing(cfg, layer, x, idx, w)
        assert _rel(y, yr.detach()) < 2e-2
        layer.release()


def test_fused_layer_module_api_trains():
    """Through MoELayer.forward (router included): loss goes down over a few SGD steps, twice the same result."""
    cfg, layer = _make_layer("gelu", 1.25, e=16, d=256, f=512, tokens=2048)
    x = (torch.randn(4, 512, cfg.d_model, device="cuda")).to(cfg.dtype)
    target = torch.randn_like(x)
    opt = torch.optim.SGD(layer.parameters(), lr=0.05)
    losses = []
    for _ in range(8):
        opt.zero_grad(set_to_none=True)
        loss = F.mse_loss(layer(x).float(), target.float())
        loss.backward()
        opt.step()
        losses.append(float(loss))
    layer._fused_impl().ctx.check_status("train loop")
    assert losses[-1] < losses[0]
    assert layer.gate.gate.weight.grad is not None and layer.gate.gate.weight.grad.abs().sum() > 0
    with torch.no_grad():
        a = layer(x)
        b = layer(x)
    assert torch.equal(a, b), "the fused path is deterministic"


def test_receive_buffer_overflow_drops_rows_consistently_and_is_reported():
    """A receive buffer that is too small: the surplus rows are dropped on both sides (no wait runs out), the
    tokens whose slots all fitted still match the oracle, and check_status raises MoEOverflow."""
    import time
    from ccfuser_b200 import MoEConfig, MoELayer, MoEOverflow
    from ccfuser_b200.ops.fused import topk_softmax, _FusedMoEFn
    torch.manual_seed(0)
    tokens = 2048
    cfg = MoEConfig(d_model=256, d_ffn=512, num_experts=4, top_k=2, capacity_factor=None, activation="gelu",
                    dtype=torch.bfloat16, ep_size=1, backend="fused", max_tokens=tokens, recv_factor=0.5)
    layer = MoELayer(cfg, device="cuda")
    with torch.no_grad():
        for p in layer.parameters():
            p.copy_(torch.randn_like(p) * 0.05)
    fm = layer._fused_impl()
    assert fm.max_rows < tokens * 2
    x = (torch.randn(tokens, 256, device="cuda") * 0.5).bfloat16()
    idx, w = topk_softmax(layer.gate.logits(x), 2)
    ex = layer.experts
    t0 = time.time()
    with torch.no_grad():
        y = _FusedMoEFn.apply(x, w, idx, ex.htoh4.weight, ex.htoh4.bias, None, None, ex.h4toh.weight, ex.h4toh.bias, fm)
    torch.cuda.synchronize()
    assert time.time() - t0 < 3.0, "an overflow must not make any wait run into its limit"
    with pytest.raises(MoEOverflow):
        fm.ctx.check_status("overflow test")
    yr, *_ = _oracle_with_routing(cfg, layer, x, idx, w)
    kept = (fm.slot_row[:tokens * 2].view(tokens, 2) >= 0).all(1)
    assert 0 < int(kept.sum()) < tokens
    assert _rel(y[kept], yr[kept].detach()) < 3e-2
    assert torch.isfinite(y.float()).all()


def test_fused_sgd_matches_torch():
    from ccfuser_b200.ops.optim import FusedSGD
    torch.manual_seed(0)
    for dtype, n in [(torch.bfloat16, 1000003), (torch.float16, 4096), (torch.bfloat16, 7)]:
        p = torch.randn(n, device="cuda").to(dtype)
        g = torch.randn(n, device="cuda").to(dtype)
        a = torch.nn.Parameter(p.clone())
        a.grad = g.clone()
        FusedSGD([a], lr=0.1, weight_decay=0.01).step()
        ref = (p.float() - 0.1 * (g.float() + 0.01 * p.float())).to(dtype)
        # fp32 arithmetic, one rounding to the parameter type (an FMA contraction may move the last bit)
        assert torch.allclose(a.detach().float(), ref.float(), rtol=8e-3, atol=1e-3)


def test_fused_sgd_many_tensors_in_few_launches():
    """More tensors than one launch takes, both dtypes, odd sizes: every tensor gets the same update as alone."""
    from ccfuser_b200 import native as N
    from ccfuser_b200.ops.optim import FusedSGD
    torch.manual_seed(1)
    sizes = [1, 7, 8, 9, 2048, 4099, 65536, 300001] * 13          # 104 tensors
    params, refs = [], []
    for i, n in enumerate(sizes):
        dtype = torch.float16 if i % 3 == 0 else torch.bfloat16
        p = torch.randn(n, device="cuda").to(dtype)
        g = torch.randn(n, device="cuda").to(dtype)
        a = torch.nn.Parameter(p.clone())
        a.grad = g.clone()
        params.append(a)
        refs.append((p.float() - 0.05 * (g.float() + 0.1 * p.float())).to(dtype))
    before = N.LAUNCHES[0]
    FusedSGD(params, lr=0.05, weight_decay=0.1).step()
    assert N.LAUNCHES[0] - before <= 4                            # 35 fp16 + 69 bf16 tensors, 48 per launch
    for a, ref in zip(params, refs):
        assert torch.allclose(a.detach().float(), ref.float(), rtol=8e-3, atol=1e-3)


def test_bounded_wait_reports_timeout_without_hanging():
    """A wait on a flag that nothing sets gives up after its limit and records a status; the context stays usable."""
    from ccfuser_b200 import native as N, MoECommTimeout
    from ccfuser_b200.ops.gemm import Workspace
    lib = N.load()
    ws = Workspace.get("cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    N.check(lib.ccf_wait_probe(flag.data_ptr(), 1, 20_000_000, ws.status.data_ptr(), N.stream_ptr()), "probe")
    torch.cuda.synchronize()
    with pytest.raises(MoECommTimeout):
        ws.check("probe")
    ws.check("probe")  # cleared
    assert torch.ones(4, device="cuda").sum().item() == 4


@pytest.mark.parametrize("act,native", [("gelu", True), ("swiglu", True), ("gelu", False)])
def test_sgd_in_the_weight_gradient_epilogue_matches_a_separate_step(act, native):
    """MoELayer.fuse_sgd against backward + FusedSGD.step on a copy of the layer: same weights after the step (up to the
    rounding of the gradient that only the separate path stores), same dx, biases and router untouched by the fusion."""
    from ccfuser_b200.ops.optim import FusedSGD
    lr, wd = 0.5, 0.01
    cfg, ref = _make_layer(act, 1.25, e=8, d=256, f=512, tokens=1024)
    _, fused = _make_layer(act, 1.25, e=8, d=256, f=512, tokens=1024)
    fused.load_state_dict(ref.state_dict())
    fused._fused_impl().native_runtime = native
    ref._fused_impl().native_runtime = native
    fused.fuse_sgd(lr, wd)
    x = (torch.randn(1000, cfg.d_model, device="cuda") * 0.5).to(cfg.dtype)
    gy = (torch.randn(1000, cfg.d_model, device="cuda") * 0.2).to(cfg.dtype)
    before = {n: p.detach().clone() for n, p in ref.named_parameters()}
    outs = []
    for layer in (ref, fused):
        xi = x.clone().requires_grad_(True)
        layer(xi).backward(gy)
        outs.append(xi.grad)
    opt = FusedSGD([p for n, p in ref.named_parameters() if n.startswith("experts.") and n.endswith("weight")], lr=lr, weight_decay=wd)
    opt.step()
    torch.cuda.synchronize()
    fused.check_status()
    assert _rel(outs[1], outs[0]) < 1e-2                      # dgrad-1 ran on the old weights
    for n, p in fused.named_parameters():
        q = dict(ref.named_parameters())[n]
        if n.startswith("experts.") and n.endswith("weight"):
            assert p.grad is None
            upd_f, upd_r = p.detach().float() - before[n].float(), q.detach().float() - before[n].float()
            assert float(upd_r.abs().max()) > 1e-3              # the step is visible at bf16 resolution
            assert _rel(upd_f, upd_r) < 5e-2, n
        else:
            assert p.grad is not None and torch.equal(p.detach(), before[n])
            assert _rel(p.grad, q.grad) < 2e-2, n
    ref.release()
    fused.release()
