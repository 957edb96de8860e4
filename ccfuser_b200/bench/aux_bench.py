"""Device-timed throughput of the memory-bound kernels around the grouped GEMMs on one GPU: router (forward and its
GEMM-free backward), LayerNorm (forward / backward), grouped column sums, slot reduce, SGD step. Each case prints one
JSON line with the achieved bytes per second against the measured copy bandwidth (MEASURED_PEAKS.json at the
repository root when present): these kernels read or write a [tokens, d] matrix once, so that is their roofline.

    python -m ccfuser_b200.bench.aux_bench --tokens 16384 --d-model 2048 --experts 64
"""
from __future__ import annotations

import argparse
import json

import torch

from .. import native as N
from .gemm_bench import measured_peaks, time_fn


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--d-ffn", type=int, default=8192)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--cases", default="router,router_bwd,layernorm,colsum,reduce,sgd")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    _, hbm, src = measured_peaks()
    dev = "cuda"
    t, d, f, e, k = args.tokens, args.d_model, args.d_ffn, args.experts, args.top_k
    lib = N.load()
    cases = args.cases.split(",")

    def report(name, nbytes, fn, **extra):
        med, best, _ = time_fn(fn, args.iters)
        rec = {"case": name, "ms_median": round(med, 4), "ms_best": round(best, 4), "algorithmic_mb": round(nbytes / 1e6, 1),
               "gb_per_s": round(nbytes / med / 1e6, 1), "frac_of_" + src + "_copy_bandwidth": round(nbytes / med / 1e6 / hbm, 3)}
        rec.update(extra)
        print(json.dumps(rec), flush=True)

    x = torch.randn(t, d, device=dev, dtype=torch.bfloat16)
    if "router" in cases or "router_bwd" in cases:
        from ..ops.router import fused_router
        wg = (torch.randn(e, d, device=dev) * 0.05).bfloat16().requires_grad_(True)
        xr = x.clone().requires_grad_(True)
        if "router" in cases:
            with torch.no_grad():
                report("router_tensor_core", t * d * 2 + e * d * 2 + t * k * 8, lambda: fused_router(x, wg, None, k))
        if "router_bwd" in cases:
            idx, w = fused_router(xr, wg, None, k)
            gw = torch.randn_like(w)

            def bwd():
                xr.grad = None
                wg.grad = None
                torch.autograd.backward(w, gw, retain_graph=True)
            # dx: writes [T, d]; dW: reads [T, d]
            report("router_backward_dx_dw", 2 * t * d * 2, bwd)
    if "layernorm" in cases:
        from ..ops.norm import LayerNorm
        ln = LayerNorm(d, device=dev, dtype=torch.bfloat16)
        xl = x.clone().requires_grad_(True)
        with torch.no_grad():
            report("layernorm_forward", 2 * t * d * 2, lambda: ln(x))
        y = ln(xl)
        gy = torch.randn_like(y)

        def ln_bwd():
            xl.grad = None
            torch.autograd.backward(y, gy, retain_graph=True)
        report("layernorm_backward", 3 * t * d * 2, ln_bwd)
        tl = torch.nn.LayerNorm(d, device=dev, dtype=torch.bfloat16)
        xt = x.clone().requires_grad_(True)
        yt = tl(xt)

        def tl_bwd():
            xt.grad = None
            torch.autograd.backward(yt, gy, retain_graph=True)
        with torch.no_grad():
            report("layernorm_forward_torch", 2 * t * d * 2, lambda: tl(x))
        report("layernorm_backward_torch", 3 * t * d * 2, tl_bwd)
    if "colsum" in cases:
        groups = 8
        rows = t * k // groups // 128 * 128
        h = torch.randn(rows * groups, f, device=dev, dtype=torch.bfloat16)
        gb = torch.arange(groups, dtype=torch.int32, device=dev) * rows
        gr = torch.full((groups,), rows, dtype=torch.int32, device=dev)
        out = torch.empty(groups, f, device=dev, dtype=torch.bfloat16)
        report("colsum_grouped", rows * groups * f * 2,
               lambda: N.check(lib.ccf_colsum_grouped(h.data_ptr(), f, f, groups, gb.data_ptr(), gr.data_ptr(), out.data_ptr(), 0,
                                                      N.stream_ptr()), "ccf_colsum_grouped"))
    if "reduce" in cases:
        comb = torch.randn(t * k, d, device=dev, dtype=torch.bfloat16)
        slot_row = torch.zeros(t * k, dtype=torch.int32, device=dev)
        y = torch.empty(t, d, device=dev, dtype=torch.bfloat16)
        report("combine_reduce", (k + 1) * t * d * 2,
               lambda: N.check(lib.ccf_combine_reduce(comb.data_ptr(), slot_row.data_ptr(), y.data_ptr(), t, k, d, 0, N.stream_ptr()),
                               "ccf_combine_reduce"))
    if "sgd" in cases:
        n = 8 * d * f
        p = torch.randn(n, device=dev, dtype=torch.bfloat16)
        g = torch.randn(n, device=dev, dtype=torch.bfloat16)
        report("sgd_step", 3 * n * 2,
               lambda: N.check(lib.ccf_sgd_step(p.data_ptr(), g.data_ptr(), n, 1e-4, 0.0, 0, N.stream_ptr()), "ccf_sgd_step"))


if __name__ == "__main__":
    main()
