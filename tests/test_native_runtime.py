"""The native layer runtime (csrc/runtime.cu) builds the same launches as the Python path: its dry-run output is compared
field by field with the launch blocks recorded from ops/fused.py. Runs without a GPU."""
import ctypes as C

import pytest
import torch

from ccfuser_b200 import MoEConfig, MoELayer
from ccfuser_b200 import native as N


@pytest.fixture(autouse=True)
def _fresh_context():
    """Layers of one process share their communication context; these tests change its mode, so each starts clean."""
    from ccfuser_b200.ops.fused import CommContext
    CommContext._instances.clear()
    yield
    CommContext._instances.clear()


def _flat(s, prefix=""):
    out = {}
    for name, _ in s._fields_:
        v = getattr(s, name)
        if isinstance(v, C.Structure):
            out.update(_flat(v, prefix + name + "."))
        elif isinstance(v, C.Array):
            out[prefix + name] = tuple(x or 0 for x in v)
        else:
            out[prefix + name] = v or 0
    return out


def _gemms(calls):
    return [N.GemmLaunch.from_buffer_copy(c[1][0]) for c in calls if c[0] == "ccf_gemm_launch"]


def _compare(py, nat, skip):
    a, b = _flat(py), _flat(nat)
    assert a.keys() == b.keys()
    diff = {k: (a[k], b[k]) for k in a if k not in skip and a[k] != b[k]}
    assert not diff, diff


def _run_case(act, bias, tokens, world=1, rank=0):
    cfg = MoEConfig(d_model=128, d_ffn=256, num_experts=4, top_k=2, activation=act, bias=bias, dtype=torch.bfloat16,
                    ep_size=world, backend="fused", max_tokens=256, capacity_factor=1.5)
    layer = MoELayer(cfg, device="cpu")
    fm = layer._fused_impl()
    fm.native_runtime = False
    real = N.load()
    x = torch.randn(tokens, 128).bfloat16().requires_grad_(True)
    # --- the Python path, launch by launch
    with N.record_launches() as rec:
        layer(x).float().sum().backward()
    py = _gemms(rec.calls)
    epoch_py = N.PlanArgs.from_buffer_copy([c for c in rec.calls if c[0] == "ccf_plan"][0][1][0]).epoch
    # --- the native path: record the two C calls it makes, then ask the real library what they would launch
    fm.native_runtime = True
    x2 = x.detach().clone().requires_grad_(True)
    with N.record_launches() as rec2:
        layer(x2).float().sum().backward()
    fm.native_runtime = False
    names = [n for n in rec2.names() if n.startswith("ccf_layer")]
    assert names == ["ccf_layer_forward", "ccf_layer_backward"]
    assert "ccf_gemm_launch" not in rec2.names() and "ccf_plan" not in rec2.names()
    fwd = [c for c in rec2.calls if c[0] == "ccf_layer_forward"][0][1]
    bwd = [c for c in rec2.calls if c[0] == "ccf_layer_backward"][0][1]
    desc = N.Layer.from_buffer_copy(fwd[0])
    buf = (N.GemmLaunch * 8)()
    cnt = C.c_int(0)
    xp, idxp, wp, yp, t, cap, save_pre, epoch = fwd[1:9]
    assert (t, cap, save_pre, epoch) == (tokens, cfg.capacity(tokens), 1, epoch_py + 1)
    assert real.ccf_layer_forward(C.byref(desc), xp, idxp, wp, yp, t, cap, save_pre, epoch, None, buf, 8, C.byref(cnt)) == 0
    nat = [N.GemmLaunch.from_buffer_copy(bytes(buf[i])) for i in range(cnt.value)]
    grads = N.LayerGrads.from_buffer_copy(bwd[4])
    cnt2 = C.c_int(0)
    assert real.ccf_layer_backward(C.byref(N.Layer.from_buffer_copy(bwd[0])), bwd[1], bwd[2], bwd[3], C.byref(grads), bwd[5],
                                   bwd[6], None, buf, 8, C.byref(cnt2)) == 0
    nat += [N.GemmLaunch.from_buffer_copy(bytes(buf[i])) for i in range(cnt2.value)]
    assert len(nat) == len(py) == (7 if act == "swiglu" else 6)
    per_call = {"args.disp.x", "args.disp.slot_expert", "args.disp.slot_gate", "args.disp.dgate"}
    outs = {"args.out0", "args.out1"}
    swiglu = act == "swiglu"
    skips = [per_call, set(), per_call | outs, {"args.out0"}] + [{"a0", "args.out0"}] * (2 if swiglu else 1) + [{"a0", "a1"}]
    for p, n, skip in zip(py, nat, skips):
        _compare(p, n, skip)
    # the per-call tensors of the native path are the ones the caller passed
    g1, dg2, dg1 = nat[0], nat[2], nat[-1]
    assert (g1.args.disp.x, g1.args.disp.slot_expert, g1.args.disp.slot_gate) == (xp, idxp, wp)
    assert (dg2.args.disp.x, dg2.args.disp.dgate, dg2.args.out0) == (bwd[1], grads.dgate, grads.dh)
    assert nat[3].args.out0 == grads.dw2 and dg1.a0 == grads.dh
    if swiglu:
        assert dg2.args.out1 == grads.dh2 and dg1.a1 == grads.dh2
        assert (nat[4].a0, nat[4].args.out0, nat[5].a0, nat[5].args.out0) == (grads.dh, grads.dwg, grads.dh2, grads.dw1)
    else:
        assert (nat[4].a0, nat[4].args.out0) == (grads.dh, grads.dw1)
    assert bool(grads.db1) == bias and bool(grads.db2) == bias and bool(grads.dbg) == (bias and swiglu)
    return True


@pytest.mark.parametrize("act,bias,tokens", [("gelu", True, 200), ("relu", False, 77), ("swiglu", True, 256),
                                             ("swiglu", False, 130)])
def test_native_runtime_builds_the_same_launches(act, bias, tokens):
    assert _run_case(act, bias, tokens)


def _two_rank(rank, world):
    return _run_case("gelu", True, 150, world, rank) and _run_case("swiglu", True, 99, world, rank)


def test_native_runtime_two_ranks():
    from tests.mp_util import run_ranks
    assert run_ranks(_two_rank, 2) == [True, True]


def test_inference_call_passes_save_pre_zero():
    cfg = MoEConfig(d_model=128, d_ffn=256, num_experts=4, top_k=2, activation="gelu", dtype=torch.bfloat16,
                    backend="fused", max_tokens=64)
    layer = MoELayer(cfg, device="cpu")
    layer._fused_impl().native_runtime = True
    with N.record_launches() as rec, torch.no_grad():
        layer(torch.randn(64, 128).bfloat16())
    call = [c for c in rec.calls if c[0] == "ccf_layer_forward"][0][1]
    assert call[7] == 0                                   # save_pre
    buf = (N.GemmLaunch * 4)()
    cnt = C.c_int(0)
    desc = N.Layer.from_buffer_copy(call[0])
    assert N.load().ccf_layer_forward(C.byref(desc), *call[1:9], None, buf, 4, C.byref(cnt)) == 0
    assert cnt.value == 2 and not buf[0].args.out1 and buf[0].args.out0


@pytest.mark.parametrize("act", ["gelu", "swiglu"])
def test_fused_sgd_launches_agree_and_update_in_place(act):
    """MoELayer.fuse_sgd: the weight-gradient GEMMs write over the weights (out0 = the parameter, lr and weight decay in
    the launch block), dgrad-1 runs before the wgrad-1 launches that overwrite what it reads, no weight gradient comes
    back; the Python path and the native runtime build the same launches in the same order."""
    cfg = MoEConfig(d_model=128, d_ffn=256, num_experts=4, top_k=2, activation=act, bias=True, dtype=torch.bfloat16,
                    ep_size=1, backend="fused", max_tokens=256)
    layer = MoELayer(cfg, device="cpu")
    layer.fuse_sgd(0.25, 0.01)
    fm = layer._fused_impl()
    ex = layer.experts
    real = N.load()
    x = torch.randn(100, 128).bfloat16().requires_grad_(True)
    fm.native_runtime = False
    with N.record_launches() as rec:
        layer(x).float().sum().backward()
    py = _gemms(rec.calls)[2:]                                  # the backward launches
    assert ex.htoh4.weight.grad is None and ex.h4toh.weight.grad is None and ex.htoh4.bias.grad is not None
    swiglu = act == "swiglu"
    # order: dgrad-2, wgrad-2 (in place on w2), dgrad-1 (COMBINE), then the wgrad-1 launches (in place on wg / w1)
    assert [g.epi for g in py] == [N.EPI_DSWIGLU if swiglu else N.EPI_DACT, N.EPI_STORE, N.EPI_COMBINE] + [N.EPI_STORE] * (2 if swiglu else 1)
    assert py[1].args.out0 == ex.h4toh.weight.data_ptr() and abs(py[1].args.sgd_lr - 0.25) < 1e-7 and abs(py[1].args.sgd_wd - 0.01) < 1e-7
    tail = [g.args.out0 for g in py[3:]]
    assert tail == ([ex.htoh4_gate.weight.data_ptr(), ex.htoh4.weight.data_ptr()] if swiglu else [ex.htoh4.weight.data_ptr()])
    assert py[0].args.sgd_lr == 0 and py[2].args.sgd_lr == 0
    # the native runtime: same blocks
    fm.native_runtime = True
    x2 = x.detach().clone().requires_grad_(True)
    with N.record_launches() as rec2:
        layer(x2).float().sum().backward()
    bwd = [c for c in rec2.calls if c[0] == "ccf_layer_backward"][0][1]
    grads = N.LayerGrads.from_buffer_copy(bwd[4])
    assert abs(grads.sgd_lr - 0.25) < 1e-7 and not grads.dw1 and not grads.dw2
    buf = (N.GemmLaunch * 8)()
    cnt = C.c_int(0)
    assert real.ccf_layer_backward(C.byref(N.Layer.from_buffer_copy(bwd[0])), bwd[1], bwd[2], bwd[3], C.byref(grads), bwd[5],
                                   bwd[6], None, buf, 8, C.byref(cnt)) == 0
    nat = [N.GemmLaunch.from_buffer_copy(bytes(buf[i])) for i in range(cnt.value)]
    assert len(nat) == len(py)
    per_call = {"args.disp.x", "args.disp.slot_expert", "args.disp.slot_gate", "args.disp.dgate", "args.out0", "args.out1"}
    for p, n, skip in zip(py, nat, [per_call, set(), {"a0", "a1"}] + [{"a0"}] * 2):
        _compare(p, n, skip)
    # a layer with replicated experts refuses (their gradients travel back to the owners)
    shadowed = type("ShadowedLayer", (), {"config": cfg.replace(shadow_experts=1), "_fused": None})()
    with pytest.raises(ValueError):
        MoELayer.fuse_sgd(shadowed, 0.1)
    layer.fuse_sgd(None)
    assert fm.sgd is None
