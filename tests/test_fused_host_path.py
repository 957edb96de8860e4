"""Host side of the fused path without a GPU: the library calls are recorded instead of run, and the sequence of
launches and their argument blocks are checked (which kernels, which operands, which epilogues)."""
import pytest
import torch

from ccfuser_b200 import MoEConfig, MoELayer
from ccfuser_b200 import native as N


@pytest.fixture(autouse=True)
def _fresh_context(monkeypatch):
    """Layers of one process share their communication context; these tests change its mode, so each starts clean.
    They look at the launches one by one, so they use the launch-by-launch Python path (the default issues a whole
    pass with one native call, which tests/test_native_runtime.py compares with this path)."""
    from ccfuser_b200.ops.fused import CommContext
    monkeypatch.setenv("CCFUSER_NATIVE_RUNTIME", "0")
    CommContext._instances.clear()
    yield
    CommContext._instances.clear()


def _layer(act="gelu", tokens=256, e=4, d=128, f=256, k=2, **kw):
    cfg = MoEConfig(d_model=d, d_ffn=f, num_experts=e, top_k=k, activation=act, dtype=torch.bfloat16, ep_size=1,
                    backend="fused", max_tokens=tokens, **kw)
    return cfg, MoELayer(cfg, device="cpu")


def _gemms(rec):
    return [N.GemmLaunch.from_buffer_copy(c[1][0]) for c in rec.calls if c[0] == "ccf_gemm_launch"]


def test_forward_backward_launch_sequence_gelu():
    cfg, layer = _layer("gelu")
    x = torch.randn(200, cfg.d_model).bfloat16().requires_grad_(True)
    with N.record_launches() as rec:
        y = layer(x)
        n_fwd = len(rec.calls)
        y.float().sum().backward()
    names = rec.names()
    assert names[:n_fwd] == ["ccf_topk_softmax", "ccf_route_ordered", "ccf_plan", "ccf_gemm_launch", "ccf_gemm_launch",
                             "ccf_combine_wait", "ccf_combine_reduce"]
    assert names[n_fwd:] == ["ccf_gemm_launch", "ccf_gemm_launch", "ccf_colsum_grouped", "ccf_gemm_launch",
                             "ccf_colsum_grouped", "ccf_gemm_launch", "ccf_combine_wait", "ccf_combine_reduce",
                             "ccf_topk_softmax_bwd"]
    fm = layer._fused_impl()
    ex = layer.experts
    g1, g2, dg2, wg2, wg1, dg1 = _gemms(rec)
    d, f, e = cfg.d_model, cfg.d_ffn, cfg.num_experts
    # GEMM-1: dispatch fused in, bias + GELU, pre-activation saved for backward
    assert (g1.epi, g1.a_major, g1.b_major, g1.kgroup) == (N.EPI_BIAS_ACT, N.MAJ_K, N.MAJ_K, 0)
    assert (g1.args.n, g1.args.k, g1.args.num_groups, g1.args.b_group_rows, g1.args.act) == (f, d, e, f, N.ACT_GELU)
    assert g1.a0 == fm.xrecv.data_ptr() and g1.b0 == ex.htoh4.weight.data_ptr() and g1.args.bias0 == ex.htoh4.bias.data_ptr()
    assert g1.args.out0 == fm.h_act.data_ptr() and g1.args.out1 == fm.h_pre.data_ptr()
    assert g1.args.tile_flags == fm.ctx.tile_flags.data_ptr() and g1.args.n_comm_ctas > 0
    assert g1.args.disp.x == x.data_ptr() and g1.args.disp.backward == 0 and g1.args.disp.top_k == 2
    assert g1.args.disp.peer_recv[0] == fm.xrecv.data_ptr() and g1.args.disp.e_total == e
    assert g1.args.disp.capacity == cfg.capacity(200) and g1.args.disp.d == d
    # GEMM-2: combine epilogue into this rank's combine buffer, finish token
    assert (g2.epi, g2.args.n, g2.args.k, g2.args.send_finish, g2.args.world) == (N.EPI_COMBINE, d, f, 1, 1)
    assert g2.a0 == fm.h_act.data_ptr() and g2.b0 == ex.h4toh.weight.data_ptr() and g2.args.peer_comb[0] == fm.comb.data_ptr()
    assert g2.args.row_gate == fm.ctx.row_gate.data_ptr() and not g2.args.tile_flags and g2.args.n_comm_ctas == 0
    # backward: dy dispatch + dgrad-2 with GELU', both wgrads k-grouped MN x MN, dgrad-1 combines into the gradient buffer
    assert (dg2.epi, dg2.b_major, dg2.args.n, dg2.args.k) == (N.EPI_DACT, N.MAJ_MN, f, d)
    assert dg2.a0 == fm.ctx.grecv.data_ptr() and dg2.b0 == ex.h4toh.weight.data_ptr() and dg2.args.aux0 == fm.h_pre.data_ptr()
    assert dg2.args.disp.backward == 1 and dg2.args.disp.saved_comb == fm.comb.data_ptr() and dg2.args.disp.dgate
    for w, a0, b0, m, n in ((wg2, fm.ctx.grecv, fm.h_act, d, f), (wg1, None, fm.xrecv, f, d)):
        assert (w.epi, w.a_major, w.b_major, w.kgroup) == (N.EPI_STORE, N.MAJ_MN, N.MAJ_MN, 1)
        assert (w.args.m_per_group, w.args.n, w.args.ld_out) == (m, n, n) and w.b0 == b0.data_ptr()
        if a0 is not None:
            assert w.a0 == a0.data_ptr()
    assert wg1.a0 == dg2.args.out0                                  # wgrad-1 reads dh written by dgrad-2
    assert (dg1.epi, dg1.b_major, dg1.args.n, dg1.args.k) == (N.EPI_COMBINE, N.MAJ_MN, d, f)
    assert dg1.a0 == dg2.args.out0 and dg1.b0 == ex.htoh4.weight.data_ptr()
    assert dg1.args.peer_comb[0] == fm.ctx.gcomb.data_ptr() and not dg1.args.row_gate and dg1.args.send_finish == 1
    # gradients come back with the right shapes
    assert ex.htoh4.weight.grad.shape == ex.htoh4.weight.shape and ex.h4toh.bias.grad.shape == ex.h4toh.bias.shape
    assert x.grad.shape == x.shape and layer.gate.gate.weight.grad is not None


def test_inference_forward_skips_pre_activation_stores_and_swiglu_operands():
    cfg, layer = _layer("swiglu", bias=False)
    x = torch.randn(100, cfg.d_model).bfloat16()
    with N.record_launches() as rec, torch.no_grad():
        layer(x)
    g1, g2 = _gemms(rec)
    ex, fm = layer.experts, layer._fused_impl()
    assert g1.epi == N.EPI_SWIGLU and g1.b0 == ex.htoh4.weight.data_ptr() and g1.b1 == ex.htoh4_gate.weight.data_ptr()
    assert g1.args.out0 == fm.h_act.data_ptr() and not g1.args.out1 and not g1.args.out2      # nothing saved for backward
    assert not g1.args.bias0 and not g1.args.bias1 and not g2.args.bias0
    x2 = x.clone().requires_grad_(True)
    with N.record_launches() as rec:
        layer(x2).float().sum().backward()
    gem = _gemms(rec)
    assert len(gem) == 2 + 5                                        # swiglu: dgrad-2, wgrad-2, two wgrad-1 halves, dgrad-1
    assert gem[0].args.out1 == fm.h_pre.data_ptr() and gem[0].args.out2 == fm.h_pre2.data_ptr()
    assert gem[2].epi == N.EPI_DSWIGLU and gem[2].args.aux0 == fm.h_pre.data_ptr() and gem[2].args.aux1 == fm.h_pre2.data_ptr()
    assert gem[6].args.kseg == 2 and gem[6].b0 == ex.htoh4_gate.weight.data_ptr() and gem[6].b1 == ex.htoh4.weight.data_ptr()
    assert "ccf_colsum_grouped" not in rec.names()                 # no biases, no bias gradients


def test_epoch_advances_and_device_epoch_switch():
    cfg, layer = _layer("relu")
    x = torch.randn(64, cfg.d_model).bfloat16()
    with N.record_launches() as rec, torch.no_grad():
        layer(x)
        layer(x)
        layer._fused_impl().ctx.use_device_epoch()
        layer(x)
    plans = [c for c in rec.calls if c[0].startswith("ccf_plan")]
    assert [c[0] for c in plans] == ["ccf_plan", "ccf_plan", "ccf_plan_dev_epoch"]
    e1, e2 = (N.PlanArgs.from_buffer_copy(c[1][0]).epoch for c in plans[:2])
    assert e2 == e1 + 1
    assert plans[2][1][1] == layer._fused_impl().ctx.epoch_dev.data_ptr()
    assert int(layer._fused_impl().ctx.epoch_dev) == e2           # the device counter starts where the host one stopped


def _two_rank_fn(rank, world):
    cfg = MoEConfig(d_model=128, d_ffn=256, num_experts=4, top_k=2, activation="gelu", dtype=torch.bfloat16,
                    ep_size=world, backend="fused", max_tokens=128)
    layer = MoELayer(cfg, device="cpu")
    x = torch.randn(100, 128).bfloat16().requires_grad_(True)
    with N.record_launches() as rec:
        layer(x).float().sum().backward()
    fm = layer._fused_impl()
    g = _gemms(rec)
    plan = N.PlanArgs.from_buffer_copy([c for c in rec.calls if c[0] == "ccf_plan"][0][1][0])
    mine = {"xrecv": fm.xrecv.data_ptr(), "comb": fm.comb.data_ptr(), "grecv": fm.ctx.grecv.data_ptr(),
            "gcomb": fm.ctx.gcomb.data_ptr(), "tile_flags": fm.ctx.tile_flags.data_ptr(), "done": fm.ctx.done.data_ptr(),
            "cnt_table": fm.ctx.cnt_table.data_ptr(), "row_src": fm.ctx.row_src.data_ptr()}
    seen = {"xrecv": list(g[0].args.disp.peer_recv)[:world], "comb": list(g[1].args.peer_comb)[:world],
            "grecv": list(g[2].args.disp.peer_recv)[:world], "gcomb": list(g[-1].args.peer_comb)[:world],
            "tile_flags": list(g[0].args.disp.peer_tile_flags)[:world], "done": list(g[1].args.peer_done)[:world],
            "cnt_table": list(plan.peer_table)[:world], "row_src": list(g[0].args.disp.peer_row_src)[:world]}
    return mine, seen, (plan.world, plan.my_rank, plan.e_loc, g[0].args.disp.my_rank, g[0].args.disp.experts_per_rank, g[1].args.world)


def test_two_rank_peer_pointers_line_up():
    """Every peer pointer a rank passes to its kernels is the address the owner itself uses for that buffer (host
    stand-in memory, addresses exchanged as numbers), and its own completion counter slot on every rank."""
    from tests.mp_util import run_ranks
    res = run_ranks(_two_rank_fn, 2)
    for r in range(2):
        mine, seen, meta = res[r]
        assert meta == (2, r, 2, r, 2, 2)
        for key in ("xrecv", "comb", "grecv", "gcomb", "tile_flags", "cnt_table", "row_src"):
            assert seen[key] == [res[0][0][key], res[1][0][key]], key
        # rank r bumps element r of every rank's `done` array
        assert seen["done"] == [res[0][0]["done"] + 4 * r, res[1][0]["done"] + 4 * r]


def test_shadow_experts_on_the_fused_host_path():
    """Replicated experts with the fused backend: their slots reach the expert-parallel kernels as expert id -1, the
    replicas run as a second, single-rank instance of the same kernels (six more GEMM launches, whose operands are the
    gathered replica weights), and both parts receive gradients (kernels recorded: shapes, dtypes and wiring only)."""
    cfg, layer = _layer("gelu", shadow_experts=1)
    x = torch.randn(120, cfg.d_model).bfloat16().requires_grad_(True)
    captured = {}
    fm = layer._fused_impl()
    orig = fm.run_experts

    def spy(xx, idx, w):
        captured["idx"] = idx.clone()
        return orig(xx, idx, w)
    fm.run_experts = spy
    with N.record_launches() as rec:
        # the recorded top-k kernel leaves its outputs uninitialised: give the router deterministic decisions instead
        fm.route = lambda xx: (torch.arange(xx.shape[0] * 2, dtype=torch.int32).view(-1, 2) % cfg.num_experts,
                               torch.full((xx.shape[0], 2), 0.5, requires_grad=True))
        y = layer(x)
        y.float().sum().backward()
    shadow = layer.last_stats["shadow_ids"].tolist()
    idx = captured["idx"]
    assert idx.dtype == torch.int32 and (idx == shadow[0]).sum() == 0 and (idx == -1).sum() == 120 * 2 // cfg.num_experts
    assert rec.names().count("ccf_gemm_launch") == 12
    gemms = _gemms(rec)
    own = {layer.experts.htoh4.weight.data_ptr(), layer.experts.h4toh.weight.data_ptr()}
    assert sum(1 for g in gemms if g.b0 in own) == 4          # GEMM-1, GEMM-2, dgrad-2, dgrad-1 of the owners' path
    replica = [g for g in gemms if g.args.num_groups == 1]
    assert len(replica) == 6 and all(g.b0 not in own for g in replica)
    assert "ccf_topk_softmax" not in rec.names() and rec.names().count("ccf_plan") == 2
    assert y.shape == x.shape and y.dtype == torch.bfloat16
    assert layer.experts.htoh4.weight.grad is not None and x.grad is not None


def test_gpt_model_with_fused_layers_host_side():
    """The model the smoke test and the benchmark run, with its MoE layers on the fused backend (kernels recorded)."""
    from ccfuser_b200.models.gpt_moe import GPTMoE, GPTMoEConfig
    c = GPTMoEConfig(vocab_size=1024, n_layer=4, n_head=4, d_model=256, d_ffn=512, seq_len=64, num_experts=8,
                     backend="fused", max_tokens=256)
    model = GPTMoE(c, device="cpu")
    ids = torch.randint(0, c.vocab_size, (4, 64))
    with N.record_launches() as rec:
        model(ids, ids.roll(-1, 1)).backward()
    n_moe = len(model.moe_layers())
    assert n_moe == 2
    assert rec.names().count("ccf_gemm_launch") == 6 * n_moe
    assert rec.names().count("ccf_plan") == n_moe and rec.names().count("ccf_topk_softmax_bwd") == n_moe
    # both layers share one communication context (same group, sizes and dtype) but own their forward buffers
    a, b = (l._fused_impl() for l in model.moe_layers())
    assert a.ctx is b.ctx and a.xrecv.data_ptr() != b.xrecv.data_ptr()
    epochs = [N.PlanArgs.from_buffer_copy(c_[1][0]).epoch for c_ in rec.calls if c_[0] == "ccf_plan"]
    assert epochs == [1, 2]
    assert all(p.grad is not None for l in model.moe_layers() for p in l.experts.parameters())


def test_canary_guards_detect_an_overrun(monkeypatch):
    from ccfuser_b200 import MoECommError
    monkeypatch.setenv("CCFUSER_CANARY", "1")
    cfg, layer = _layer("gelu")
    fm = layer._fused_impl()
    assert fm.ctx.guard == 1024 and len(fm.ctx.buf._guards) == 9 and len(fm.buf._guards) == 2
    layer.check_status()                                            # clean
    # a write one element past the end of the forward receive buffer
    end = fm.off_xrecv + fm.max_rows * cfg.d_model * 2
    fm.buf.local[end] = 0
    with pytest.raises(MoECommError, match="guard region"):
        layer.check_status()


def test_device_barrier_arguments():
    cfg, layer = _layer("gelu")
    cc = layer._fused_impl().ctx
    with N.record_launches() as rec:
        cc.device_barrier()
        cc.device_barrier()
    a, b = (N.BarrierArgs.from_buffer_copy(c[1][0]) for c in rec.calls)
    assert rec.names() == ["ccf_flag_barrier"] * 2
    assert (a.world, a.my_rank, a.epoch, b.epoch) == (1, 0, 1, 2)
    assert a.peer_flag[0] == cc.buf.peer_ptr(0, cc.off["bar_flag"]) and a.status == cc.ws.status.data_ptr()


def _rebalance_bf16_fn(rank, world):
    import torch.distributed as dist
    cfg = MoEConfig(d_model=128, d_ffn=256, num_experts=4, top_k=2, activation="swiglu", dtype=torch.bfloat16,
                    ep_size=world, backend="fused", max_tokens=128)
    layer = MoELayer(cfg, device="cpu")
    fm = layer._fused_impl()
    desc_before = bytes(fm.native_desc())
    w = layer.experts.htoh4_gate.weight.detach().clone()
    allw = [torch.empty_like(w) for _ in range(world)]
    dist.all_gather(allw, w.float().contiguous().to(torch.float32).bfloat16())
    gate_before = layer.gate.gate.weight.detach().clone()
    placement = [3, 1, 2, 0]                                      # experts 0 and 3 swap ranks
    layer.rebalance(placement)
    full = torch.cat(allw, 0)
    want = full[torch.tensor(placement)][rank * 2:(rank + 1) * 2]
    ok_w = torch.equal(layer.experts.htoh4_gate.weight.detach(), want)
    ok_g = torch.equal(layer.gate.gate.weight.detach(), gate_before[torch.tensor(placement)])
    return ok_w, ok_g, bytes(fm.native_desc()) == desc_before


def test_bf16_experts_migrate_between_ranks_and_kernel_pointers_stay_valid():
    from tests.mp_util import run_ranks
    assert run_ranks(_rebalance_bf16_fn, 2) == [(True, True, True)] * 2


def test_memory_estimate_matches_what_the_layer_allocates():
    cfg, layer = _layer("swiglu", tokens=256, e=4, d=128, f=256)
    fm = layer._fused_impl()
    est = cfg.memory_estimate(layers=1, training=True)
    params = sum(p.numel() * p.element_size() for p in layer.parameters())
    assert est["parameters"] == params == est["gradients"]
    sym_layer = fm.max_rows * cfg.d_model * 2 + fm.max_slots * cfg.d_model * 2
    acts = sum(t.numel() * t.element_size() for t in (fm.h_act, fm.h_pre, fm.h_pre2))
    assert abs(est["layer_buffers"] - (sym_layer + acts)) < 16 * 1024            # index arrays are the remainder
    assert est["group_buffers"] >= fm.ctx.grecv.numel() * 2 + fm.ctx.gcomb.numel() * 2
    big = MoEConfig(d_model=4096, d_ffn=14336, num_experts=64, top_k=2, capacity_factor=1.2, activation="swiglu",
                    bias=False, ep_size=8, max_tokens=16384)
    total_gb = big.memory_estimate(layers=1)["total"] / 2 ** 30
    assert 8 < total_gb < 20                                                     # one Mixtral-size layer per rank


def test_fp32_router_with_half_precision_experts():
    """router_dtype=float32: the router's parameters and logits stay fp32 on every backend; on the fused path the top-k
    kernel is given fp32 logits and the one-kernel router (which needs matching operand types) is not chosen."""
    cfg, layer = _layer("gelu", router_dtype=torch.float32)
    assert layer.gate.gate.weight.dtype == torch.float32 and layer.experts.htoh4.weight.dtype == torch.bfloat16
    fm = layer._fused_impl()
    fm.fused_router = True
    x = torch.randn(64, cfg.d_model).bfloat16().requires_grad_(True)
    with N.record_launches() as rec:
        layer(x).float().sum().backward()
    topk = [c for c in rec.calls if c[0] == "ccf_topk_softmax"][0][1]
    assert topk[1] == 0 and topk[2] == 1                       # fp16 flag off, fp32 flag on
    assert "ccf_router_topk" not in rec.names()
    assert layer.gate.gate.weight.grad.dtype == torch.float32 and x.grad.dtype == torch.bfloat16
    # CPU backend with the same mixed setting against an fp32-router oracle decision
    cfg2 = cfg.replace(backend="cpu")
    l2 = MoELayer(cfg2, device="cpu")
    y = l2(torch.randn(10, cfg.d_model).bfloat16())
    assert y.dtype == torch.bfloat16 and torch.isfinite(y.float()).all()


def test_token_mask_reaches_the_kernels_as_unrouted_slots():
    cfg, layer = _layer("gelu")
    fm = layer._fused_impl()
    seen = {}
    orig = fm.run_experts
    fm.run_experts = lambda xx, idx, w: (seen.setdefault("idx", idx.clone()), orig(xx, idx, w))[1]
    fm.route = lambda xx: (torch.ones(xx.shape[0], 2, dtype=torch.int32), torch.full((xx.shape[0], 2), 0.5))
    mask = torch.tensor([True] * 30 + [False] * 10)
    with N.record_launches(), torch.no_grad():
        layer(torch.randn(40, cfg.d_model).bfloat16(), token_mask=mask)
    assert seen["idx"].dtype == torch.int32 and (seen["idx"][30:] == -1).all() and (seen["idx"][:30] == 1).all()


def test_second_forward_before_backward_raises_instead_of_corrupting():
    """One set of saved activations per layer: a forward while a backward is still owed raises; after the backward, or
    once the first result has been dropped, the layer can be called again."""
    cfg, layer = _layer("gelu")
    x = torch.randn(100, cfg.d_model).bfloat16().requires_grad_(True)
    with N.record_launches():
        y1 = layer(x)
        with pytest.raises(RuntimeError, match="previous forward"):
            layer(x)
        with pytest.raises(RuntimeError, match="previous forward"), torch.no_grad():
            layer(x)                                   # an evaluation pass in between would overwrite them as well
        y1.float().sum().backward()
        y2 = layer(x)                                  # backward has run: fine
        del y2                                         # dropped without a backward: the claim ends with its graph
        import gc
        gc.collect()
        y3 = layer(x)
        y3.float().sum().backward()
        with torch.no_grad():
            layer(x)
            layer(x)                                   # inference calls never hold a claim
