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
