"""Configuration arithmetic and the roofline helper (CPU)."""
import math

import pytest
import torch

from ccfuser_b200 import MoEConfig, zipf_router_bias
from ccfuser_b200.bench.roofline import layer_flops, nvlink_bytes, roofline


def test_capacity_and_receive_bounds():
    c = MoEConfig(d_model=64, d_ffn=128, num_experts=64, top_k=2, capacity_factor=1.2, ep_size=8, max_tokens=16384)
    assert c.experts_per_rank == 8
    assert c.capacity(16384) == math.ceil(1.2 * 16384 * 2 / 64) == 615
    # per expert: 8 sources x 615 rows, padded to 128 -> 4992; 8 local experts
    assert c.max_recv_rows() == 8 * 4992
    n = MoEConfig(d_model=64, d_ffn=128, num_experts=8, top_k=2, capacity_factor=None, ep_size=1, max_tokens=1000)
    assert n.capacity(1000) == 2000
    assert n.max_recv_rows() % 128 == 0 and n.max_recv_rows() >= 2000
    with pytest.raises(ValueError):
        MoEConfig(d_model=64, d_ffn=128, num_experts=10, ep_size=4)
    with pytest.raises(ValueError):
        MoEConfig(d_model=64, d_ffn=128, num_experts=8, activation="tanh")


def test_zipf_bias_orders_expert_popularity():
    b = zipf_router_bias(64, 1.2, 1.0, seed=0)
    p = torch.softmax(b, 0)
    top = torch.sort(p, descending=True).values
    # p_k ~ k^-1.2: the ratio of the two most popular experts is 2^1.2
    assert abs(float(top[0] / top[1]) - 2 ** 1.2) < 1e-3
    assert abs(float(p.sum()) - 1) < 1e-6


def test_roofline_numbers_for_the_large_layer():
    # 16384 tokens/GPU, top-2, SwiGLU 4096 -> 14336 -> 4096: 34.6 TFLOP per GPU forward + backward
    fl = layer_flops(16384, 4096, 14336, 2, "swiglu")
    assert abs(fl / 1e12 - 34.6) < 0.1
    by = nvlink_bytes(16384, 4096, 2, 8)
    assert abs(by / 1e6 - 4 * 268.4 * 7 / 8) < 1.0
    r = roofline(16384, 4096, 14336, 2, "swiglu", 8, peak_tflops=1675.7)
    assert r["bound"] == "compute" and abs(r["target_ms"] - 20.7) < 0.1
    small = roofline(128, 4096, 14336, 2, "swiglu", 8, backward=False, peak_tflops=1675.7, experts_per_gpu=1, hbm_gbs=6557.0)
    # one expert's weights are 352 MB: reading them (54 us) costs as much as the 256 routed rows' FLOPs
    assert abs(small["hbm_weights_ms"] - 0.0537) < 0.001 and small["target_ms"] < 0.06


def test_plot_tool_writes_wellformed_svg(tmp_path):
    """The figure tool reads the experiment CSVs (its own and the reference's recorded format with a partial
    num_expert column) and writes parseable SVG."""
    import xml.etree.ElementTree as ET
    from ccfuser_b200.bench import plot
    d = tmp_path / "data"
    d.mkdir()
    (d / "moe_layer_t.csv").write_text("name,num_expert,total_time,forward_time,backward_time\\n\n"
                                       "a,4,2.0,1.0,1.0\na,8,2.5,1.2,1.3\nb,4,9.0,4.0,5.0\nb,8,9.5,4.5,5.0\n")
    (d / "e2e_model_t.csv").write_text("name,MOE-GPT,MOE-BERT\nnaive,10,20\nfused,12,25\n")
    (d / "kernel_eval_expert_t.csv").write_text(
        "kernel, locality, time, all2all, num_expert\nAG, 0.25, 0.2, 0 \nAll2All-GEMM, 0.25, 0.5, 0.1\n"
        "GA, 0.25, 0.2, 0 \nGEMM-All2All, 0.25, 0.4, 0.1, 2\n")
    made = plot.main(["--data", str(d), "--out", str(tmp_path / "fig")])
    assert len(made) == 3 + 1 + 2
    for p in made:
        root = ET.parse(p).getroot()
        assert root.tag.endswith("svg") and len(list(root.iter())) > 20


def test_expert_parallel_group_must_share_a_machine():
    import pytest
    from ccfuser_b200.parallel.symm import check_same_host, host_id
    check_same_host([host_id()] * 8)
    with pytest.raises(RuntimeError, match="one machine"):
        check_same_host(["node-a/1", "node-a/1", "node-b/2", "node-b/2"])


def test_import_of_a_reference_state_dict_drops_the_shadow_slots():
    import torch
    from ccfuser_b200 import MoEConfig, MoELayer
    from ccfuser_b200.utils.checkpoint import import_reference_state
    layer = MoELayer(MoEConfig(d_model=16, d_ffn=32, num_experts=4, dtype=torch.float32, backend="cpu"))
    ref = {k: (torch.cat([v, torch.randn(3, *v.shape[1:])], 0) if k.startswith("experts.") else v.clone())
           for k, v in layer.state_dict().items()}
    assert ref["experts.htoh4.weight"].shape == (7, 32, 16)
    state = import_reference_state(ref, 4)
    layer.load_state_dict(state)
    assert torch.equal(layer.experts.htoh4.weight, ref["experts.htoh4.weight"][:4])


def test_native_entry_points_reject_bad_arguments_before_touching_the_device():
    import ctypes as C
    from ccfuser_b200 import native as N
    lib = N.load()
    ok = dict(tokens=128, d=256, e=64, k=2)

    def router(**kw):
        a = dict(ok, **kw)
        return lib.ccf_router_topk(None, None, None, a["tokens"], a["d"], a["e"], a["k"], 0, None, None, None, None, 0, -1, None)
    assert router(e=257) == -2 and router(k=9) == -2 and router(k=3, e=2) == -2 and router(d=32) == -2
    assert router(d=260) == -2 and router(tokens=0) == -2
    b = N.BarrierArgs()
    b.world, b.my_rank = 9, 0
    assert lib.ccf_flag_barrier(C.byref(b), None) == -2
    b.world, b.my_rank = 4, 4
    assert lib.ccf_flag_barrier(C.byref(b), None) == -2
    assert lib.ccf_layer_forward(None, None, None, None, None, 0, 0, 0, 0, None, None, 0, None) == -2
    layer = N.Layer()
    layer.world = 0
    assert lib.ccf_layer_forward(C.byref(layer), None, None, None, None, 0, 0, 0, 0, None, None, 0, None) == -2
    p = N.PlanArgs()
    p.e_total, p.world = 300, 2
    assert lib.ccf_plan(C.byref(p), None) == -2


def test_router_selection_rule_on_the_host():
    """The one-kernel router's epilogue rule (running top-8 with stable ties, softmax over the first k), compiled for
    the host from the same source, against the reference top-k + softmax."""
    import torch
    from ccfuser_b200 import native as N
    from ccfuser_b200.gates import topk_softmax_reference
    lib = N.load()
    g = torch.Generator().manual_seed(3)
    for t, e, k in ((300, 8, 2), (257, 64, 2), (100, 200, 8), (64, 256, 4), (50, 5, 5), (10, 1, 1)):
        logits = torch.randn(t, e, generator=g)
        logits[::7] = torch.round(logits[::7] * 2) / 2            # many exact ties
        logits[3] = 0.25                                           # a row of all-equal logits
        idx = torch.empty(t, k, dtype=torch.int32)
        w = torch.empty(t, k, dtype=torch.float32)
        assert lib.ccf_router_select_host(logits.contiguous().data_ptr(), t, e, k, idx.data_ptr(), w.data_ptr()) == 0
        ridx, rw = topk_softmax_reference(logits, k)
        assert torch.equal(idx.long(), ridx)
        assert torch.allclose(w, rw, atol=1e-6)


def test_ae_harness_writes_the_reference_csv_columns(tmp_path, monkeypatch):
    """The evaluation harness with its child runs replaced by canned records: file names and columns as the reference's
    recorded data (moe_layer_*.csv, kernel_eval_*.csv, e2e_model_*.csv), and the figure tool accepts them."""
    import csv
    from ccfuser_b200.bench import ae, plot

    def fake(gpus, module, args, port, timeout=1800):
        if module.endswith("layer_bench"):
            return [{"backend": b, "experts_per_gpu": e, "total_ms": 2.0 * f, "fwd_ms": 0.8 * f, "bwd_ms": 1.2 * f}
                    for b, f in (("fused", 1.0), ("nccl", 4.0)) for e in (4, 8)]
        if module.endswith("kernel_bench"):
            return [{"experts_per_gpu": 16, "remote_frac": rf, "fused_ag_ms": 0.25, "nccl_a2a_gemm1_ms": 2.0, "nccl_a2a_in_ms": 0.1,
                     "fused_ga_ms": 0.2, "gemm2_nccl_a2a_ms": 1.9, "nccl_a2a_out_ms": 0.1} for rf in (0.45, 0.25)]
        return [{"step_ms": 33.0}]
    monkeypatch.setattr(ae, "torchrun", fake)
    p10, _ = ae.fig10(4, str(tmp_path), 3)
    p12, _ = ae.fig12(4, str(tmp_path), 3)
    p11, _ = ae.fig11(4, str(tmp_path), 3)
    rows = list(csv.reader(open(p10)))
    assert rows[0] == ["name", "num_expert", "total_time", "forward_time", "backward_time"] and len(rows) == 5
    assert rows[1][0] == "ccfuser_b200" and rows[3][0] == "nccl_a2a"
    assert list(csv.reader(open(p12[0])))[0] == ["kernel", "locality", "time", "all2all"]
    assert list(csv.reader(open(p12[1])))[0] == ["kernel", "locality", "time", "all2all", "num_expert"]
    e2e = list(csv.reader(open(p11)))
    assert e2e[0] == ["name", "MOE-GPT", "MOE-BERT", "MOE-Transformer-xl"] and [r[0] for r in e2e[1:]] == ["naive", "nccl_a2a", "ccfuser_b200"]
    made = plot.main(["--data", str(tmp_path), "--out", str(tmp_path / "fig")])
    assert len(made) == 3 + 1 + 2 + 2


def test_per_kernel_estimates():
    from ccfuser_b200.bench.roofline import kernel_estimates
    few = kernel_estimates(16384, 2048, 8192, 8, "gelu", peak_tflops=1392.0, hbm_gbs=6557.0)
    many = kernel_estimates(16384, 2048, 8192, 64, "gelu", peak_tflops=1392.0, hbm_gbs=6557.0)
    assert all(few[k]["bound"] == "compute" for k in few if k != "total_ms")
    assert abs(few["gemm2+combine"]["ms"] - 2 * 16384 * 2048 * 8192 / 1392e9) < 1e-3
    # with 64 experts on one GPU the weights alone make the first GEMM of each pass memory-bound
    assert many["dispatch+gemm1"]["bound"] == "hbm" and many["total_ms"] > few["total_ms"]
    sw = kernel_estimates(16384, 4096, 14336, 8, "swiglu", peak_tflops=1392.0, hbm_gbs=6557.0)
    assert abs(sw["dispatch+gemm1"]["compute_ms"] - 2 * sw["gemm2+combine"]["compute_ms"]) < 1e-3


def test_stage_timer_on_the_host():
    import time
    from ccfuser_b200.utils.tracing import StageTimer, nvtx_range
    t = StageTimer()
    for _ in range(3):
        with t.stage("sleep"):
            time.sleep(0.01)
        with t.stage("noop"), nvtx_range("x"):
            pass
    s = t.summary()
    assert set(s) == {"sleep", "noop"} and s["sleep"] >= 9.0 > s["noop"]


def test_trace_analysis_on_a_synthetic_trace():
    import torch
    from ccfuser_b200.bench.overlap_trace import analyze
    ctas, slots, kblocks = 4, 6, 32
    t = torch.zeros(ctas, slots, 8, dtype=torch.int64)
    for c in range(ctas):
        t[c, slots - 1, 0] = 1000                                  # kernel start
        clk = 1000
        for i in range(3):                                         # three tiles per CTA
            t[c, i, 0] = clk; t[c, i, 1] = clk + 50; t[c, i, 2] = clk + 400      # noqa: E702
            t[c, i, 3] = clk + 100                                 # accumulator free 100 clk after the previous commit
            t[c, i, 4] = clk + 300
            t[c, i, 5] = clk + 300 + 20480                         # main loop at 80 % of the ideal 16384
            t[c, i, 6] = t[c, i, 5] + 10
            t[c, i, 7] = t[c, i, 6] + 6000
            clk = int(t[c, i, 5])
    r = analyze(t, kblocks, leaders_only=False)
    assert r["tiles"] == 12 and r["main_loop_clk"] == 20480 and r["main_loop_efficiency"] == 0.8
    assert r["acc_wait_clk"] == 100 and r["rows_wait_clk"] == 50 and r["epilogue_clk"] == 6000
    assert analyze(torch.zeros(2, 3, 8, dtype=torch.int64), 8)["tiles"] == 0


def test_status_words_are_explained():
    import torch
    from ccfuser_b200 import MoECommTimeout
    from ccfuser_b200.ops.gemm import Workspace, describe_status
    assert "rank 3" in describe_status(2, 0x800003) and "count exchange" in describe_status(2, 0x800003)
    assert "owner rank 5" in describe_status(2, 0x400005)
    assert "tile 7" in describe_status(2, 7) and "rows 896..1023" in describe_status(2, 7)
    assert "free accumulator" in describe_status(1, 4) and "CTA-pair" in describe_status(1, 0x25)
    ws = Workspace(torch.device("cpu"))
    ws.status[0] = (0x400002 << 8) | 2
    try:
        ws.check("step 12")
        raise AssertionError("expected a time-out")
    except MoECommTimeout as e:
        assert "owner rank 2" in str(e) and "step 12" in str(e)
    assert int(ws.status[0]) == 0                                  # cleared after reporting


def test_environment_report():
    from ccfuser_b200.utils.doctor import report
    r = report()
    assert {"torch", "cuda_available", "library", "gpus", "problems"} <= set(r)
    assert r["library"]["path"].endswith("libccfuser_b200.so")
    if not r["cuda_available"]:
        assert any("no CUDA device" in p for p in r["problems"])
