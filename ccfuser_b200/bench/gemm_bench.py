"""Device-timed throughput of the tcgen05 grouped GEMM variants on one GPU (CUDA events, L2 flushed
between timed launches). Prints one JSON line per case with achieved TFLOP/s and the fraction of the
measured cuBLAS bf16 peak (MEASURED_PEAKS.json at the repository root when present)."""
from __future__ import annotations

import argparse
import json
import os

import torch

from .. import native as N
from ..ops import gemm as G


def measured_peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return d.get("bf16_tflops", 1590.0), d.get("hbm_gbs", 6650.0), "measured"
    except Exception:
        return 1590.0, 6650.0, "fallback"


def measured_sustained_tflops(default: float = 1400.0) -> float:
    """cuBLAS bf16 rate of a seconds-long back-to-back loop under the power cap (MEASURED_PEAKS.json): the applicable
    ceiling for kernels timed inside a long step, as opposed to the burst rate of a single isolated launch."""
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f).get("bf16_tflops_sustained", default))
    except Exception:
        return default


def time_fn(fn, iters=10, warmup=3, flush_mb=256, back_to_back=0):
    """Median and best time of one launch (L2 flushed before each). With ``back_to_back`` = n > 0 also the time per
    launch of n launches issued without a gap (what the kernel sustains inside a long step under the power cap)."""
    flush = torch.empty(flush_mb * 1024 * 1024, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    b2b = None
    if back_to_back > 0:
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(back_to_back):
            fn()
        e.record()
        torch.cuda.synchronize()
        b2b = s.elapsed_time(e) / back_to_back
    return times[len(times) // 2], times[0], b2b


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cases", default="square,fwd1,fwd2,dgrad,dgrad_plain,wgrad,cublas",
                    help="comma-separated; also fwd1_parts and wgrad_sgd")
    ap.add_argument("--rows", type=int, default=4096 * 8)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--d", type=int, default=4096)
    ap.add_argument("--f", type=int, default=14336)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--trace", action="store_true",
                    help="add per-tile clock statistics (main-loop time against its ideal, accumulator wait, epilogue time)")
    ap.add_argument("--out", default="", help="optional JSON file for the records")
    ap.add_argument("--back-to-back", type=int, default=0,
                    help="also time this many launches of each case without gaps and report the SM clock seen meanwhile")
    args = ap.parse_args()
    from ..utils.clocks import ClockSampler, visible_index
    sampler = ClockSampler(visible_index(torch.cuda.current_device()), period=0.02)
    sampler.start()
    peak, _, src = measured_peaks()
    dev = "cuda"
    e, d, f = args.experts, args.d, args.f
    rows_per = args.rows // e
    gb = torch.arange(e, dtype=torch.int32, device=dev) * rows_per
    gr = torch.full((e,), rows_per, dtype=torch.int32, device=dev)
    r = rows_per * e
    out = []

    def report(name, flops, fn, kblocks=0):
        """fn() launches the case; if it accepts ``trace=`` and --trace is given, one more launch records per-tile clocks."""
        m0 = sampler.mark()
        med, best, b2b = time_fn(fn, args.iters, back_to_back=args.back_to_back)
        G.Workspace.get(dev).check(name)
        clk = sampler.summary_between(m0, sampler.mark())
        rec = {"case": name, "ms_median": round(med, 4), "ms_best": round(best, 4),
               "tflops_median": round(flops / med / 1e9, 1), "frac_of_" + src + "_cublas_peak": round(flops / med / 1e9 / peak, 3),
               "frac_of_" + src + "_cublas_sustained": round(flops / med / 1e9 / measured_sustained_tflops(), 3)}
        rec["clocks"] = clk
        if b2b is not None:
            rec["ms_back_to_back"] = round(b2b, 4)
            rec["tflops_back_to_back"] = round(flops / b2b / 1e9, 1)
            if clk.get("sm_mhz"):
                # tensor-pipe use implied by the clock that was seen: 148 SMs x 8192 dense bf16 FLOP per clock
                rec["frac_of_pipe_at_seen_clock"] = round(flops / b2b / 1e9 / (148 * 8192 * clk["sm_mhz"] * 1e-6), 3)
        if args.trace and kblocks > 0:
            from .overlap_trace import analyze
            tr = torch.zeros(148, 128, 8, dtype=torch.int64, device=dev)
            fn(trace=tr)
            torch.cuda.synchronize()
            rec["per_tile"] = analyze(tr, kblocks)
        print(json.dumps(rec), flush=True)
        out.append(rec)

    def gemm(**kw):
        return lambda trace=None: G.launch(trace=trace, **kw)

    cases = args.cases.split(",")
    if "square" in cases:
        m = 8192
        x = torch.randn(m, m, device=dev, dtype=torch.bfloat16)
        w = torch.randn(m, m, device=dev, dtype=torch.bfloat16)
        report("square_8192_ours", 2 * m ** 3, lambda: G.linear(x, w))
        if "cublas" in cases:
            report("square_8192_cublas", 2 * m ** 3, lambda: torch.matmul(x, w.t()))
        del x, w
    x = torch.randn(r, d, device=dev, dtype=torch.bfloat16)
    w1 = torch.randn(e, f, d, device=dev, dtype=torch.bfloat16) * 0.02
    h = torch.empty(r, f, device=dev, dtype=torch.bfloat16)
    pre = torch.empty(r, f, device=dev, dtype=torch.bfloat16)
    if "fwd1" in cases:
        report("fwd1_gelu", 2 * r * d * f, gemm(
            a0=x, b0=w1.view(e * f, d), a_major=N.MAJ_K, b_major=N.MAJ_K, epi=N.EPI_BIAS_ACT, n=f, k=d,
            group_base=gb, group_rows=gr, num_groups=e, b_group_rows=f, out0=h, out1=pre, act=N.ACT_GELU), kblocks=(d + 63) // 64)
    # the same GEMM with parts of its epilogue taken away: which part costs the main loop its efficiency
    if "fwd1_parts" in cases:
        common = dict(a0=x, b0=w1.view(e * f, d), a_major=N.MAJ_K, b_major=N.MAJ_K, epi=N.EPI_BIAS_ACT, n=f, k=d,
                      group_base=gb, group_rows=gr, num_groups=e, b_group_rows=f, out0=h)
        report("fwd1_one_output_no_act", 2 * r * d * f, gemm(act=N.ACT_NONE, **common), kblocks=(d + 63) // 64)
        report("fwd1_one_output_gelu", 2 * r * d * f, gemm(act=N.ACT_GELU, **common), kblocks=(d + 63) // 64)
        report("fwd1_two_outputs_no_act", 2 * r * d * f, gemm(act=N.ACT_NONE, out1=pre, **common), kblocks=(d + 63) // 64)
        report("fwd1_two_outputs_relu", 2 * r * d * f, gemm(act=N.ACT_RELU, out1=pre, **common), kblocks=(d + 63) // 64)
    w2 = torch.randn(e, d, f, device=dev, dtype=torch.bfloat16) * 0.02
    y = torch.empty(r, d, device=dev, dtype=torch.bfloat16)
    if "fwd2" in cases:
        report("fwd2_store", 2 * r * d * f, gemm(
            a0=h, b0=w2.view(e * d, f), a_major=N.MAJ_K, b_major=N.MAJ_K, epi=N.EPI_STORE, n=d, k=f,
            group_base=gb, group_rows=gr, num_groups=e, b_group_rows=d, out0=y), kblocks=(f + 63) // 64)
    if "dgrad" in cases:
        report("dgrad2_dact", 2 * r * d * f, gemm(
            a0=y, b0=w2.view(e * d, f), a_major=N.MAJ_K, b_major=N.MAJ_MN, epi=N.EPI_DACT, n=f, k=d,
            group_base=gb, group_rows=gr, num_groups=e, b_group_rows=d, out0=h, aux0=pre, act=N.ACT_GELU), kblocks=(d + 63) // 64)
    if "dgrad_plain" in cases:
        report("dgrad2_plain_store", 2 * r * d * f, gemm(
            a0=y, b0=w2.view(e * d, f), a_major=N.MAJ_K, b_major=N.MAJ_MN, epi=N.EPI_STORE, n=f, k=d,
            group_base=gb, group_rows=gr, num_groups=e, b_group_rows=d, out0=h), kblocks=(d + 63) // 64)
    # few rows per expert (many experts on one GPU): the one-CTA kernel, as the layer chooses there
    wgrad_two_cta = None if rows_per > 512 else False
    if "wgrad" in cases:
        dw = torch.empty(e, d, f, device=dev, dtype=torch.bfloat16)
        report("wgrad2", 2 * r * d * f, gemm(
            a0=y, b0=h, a_major=N.MAJ_MN, b_major=N.MAJ_MN, epi=N.EPI_STORE, n=f, kgroup=True, m_per_group=d,
            group_base=gb, group_rows=gr, num_groups=e, out0=dw, ld_out=f, two_cta=wgrad_two_cta), kblocks=(rows_per + 63) // 64)
        del dw
    if "wgrad_sgd" in cases:
        # the same product with the SGD step in its epilogue: w2 is read and rewritten in place, no gradient is stored
        y.normal_()
        h.normal_()
        report("wgrad2_sgd_in_place", 2 * r * d * f, gemm(
            a0=y, b0=h, a_major=N.MAJ_MN, b_major=N.MAJ_MN, epi=N.EPI_STORE, n=f, kgroup=True, m_per_group=d,
            group_base=gb, group_rows=gr, num_groups=e, out0=w2, ld_out=f, two_cta=wgrad_two_cta, sgd=(1e-6, 0.0)),
            kblocks=(rows_per + 63) // 64)
    sampler.stop()
    if args.out:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "w") as fh:
            json.dump(out, fh, indent=1)


if __name__ == "__main__":
    main()
