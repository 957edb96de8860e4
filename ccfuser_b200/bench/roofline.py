"""Roofline arithmetic for the MoE layer: target time = the slower of (FLOPs / measured GEMM peak) and
(bytes that must cross NVLink / link bandwidth); fraction = target / measured.

    python -m ccfuser_b200.bench.roofline --tokens 16384 --d-model 4096 --d-ffn 14336 --top-k 2 --act swiglu \
        --gpus 8 --measured-ms 34.9

The denominators default to the values measured on this machine type (cuBLAS bf16 burst rate from
MEASURED_PEAKS.json when present, peer-copy bandwidth 770 GB/s per direction).
"""
from __future__ import annotations

import argparse
import json

from .gemm_bench import measured_peaks, measured_sustained_tflops

NVLINK_GBS = 770.0


def layer_flops(tokens: int, d_model: int, d_ffn: int, top_k: int, act: str, backward: bool = True,
                kept_fraction: float = 1.0) -> float:
    """FLOPs of one rank's share of an expert-parallel MoE FFN call (balanced routing)."""
    mats = 3 if act == "swiglu" else 2
    fwd = 2.0 * mats * d_model * d_ffn * tokens * top_k * kept_fraction
    return fwd * (3 if backward else 1)


def nvlink_bytes(tokens: int, d_model: int, top_k: int, gpus: int, backward: bool = True, elem: int = 2,
                 kept_fraction: float = 1.0) -> float:
    """Bytes one rank sends over NVLink per call: dispatch + combine (and their mirrors in backward)."""
    remote = (gpus - 1) / gpus if gpus > 1 else 0.0
    one_way = tokens * top_k * kept_fraction * d_model * elem * remote
    return one_way * (4 if backward else 2)


def weight_bytes(d_model: int, d_ffn: int, act: str, experts_per_gpu: int, backward: bool = True, elem: int = 2) -> float:
    """HBM traffic of the expert weights alone: read once in forward; in backward read again (dgrad) and the weight
    gradients written once. With few tokens per expert this, not the FLOPs, bounds the layer."""
    mats = 3 if act == "swiglu" else 2
    w = experts_per_gpu * mats * d_model * d_ffn * elem
    return w * (3 if backward else 1)


def roofline(tokens, d_model, d_ffn, top_k, act, gpus, backward=True, kept_fraction=1.0, peak_tflops=None,
             nvlink_gbs=NVLINK_GBS, experts_per_gpu=0, hbm_gbs=None):
    if peak_tflops is None:
        peak_tflops, hbm_meas, src = measured_peaks()
    else:
        hbm_meas, src = 6557.0, "given"
    hbm_gbs = hbm_gbs or hbm_meas
    fl = layer_flops(tokens, d_model, d_ffn, top_k, act, backward, kept_fraction)
    by = nvlink_bytes(tokens, d_model, top_k, gpus, backward, kept_fraction=kept_fraction)
    t_compute = fl / (peak_tflops * 1e9)            # ms
    t_link = by / (nvlink_gbs * 1e6)                # ms
    t_hbm = weight_bytes(d_model, d_ffn, act, experts_per_gpu, backward) / (hbm_gbs * 1e6) if experts_per_gpu else 0.0
    terms = {"compute": t_compute, "nvlink": t_link, "hbm_weights": t_hbm}
    bound = max(terms, key=terms.get)
    return {"flops": fl, "nvlink_bytes": by, "compute_ms": t_compute, "link_ms": t_link, "hbm_weights_ms": t_hbm,
            "target_ms": terms[bound], "bound": bound, "peak_source": src, "peak_tflops": peak_tflops}


def kernel_estimates(rows: int, d_model: int, d_ffn: int, experts_per_gpu: int, act: str = "gelu", peak_tflops: float = None,
                     hbm_gbs: float = None, elem: int = 2):
    """Expected duration of each GEMM launch of one forward + backward pass on one rank that processes ``rows`` routed
    rows: the slower of FLOPs at the sustained GEMM rate and the launch's compulsory HBM traffic (operands read once,
    outputs written once) at the measured copy rate. To be written down before a measurement; the gap is the signal."""
    if peak_tflops is None:
        peak_tflops = measured_sustained_tflops()
    if hbm_gbs is None:
        hbm_gbs = measured_peaks()[1]
    g = 2 if act == "swiglu" else 1                 # up-projection matrices
    w1 = experts_per_gpu * g * d_model * d_ffn * elem
    w2 = experts_per_gpu * d_model * d_ffn * elem
    x, h = rows * d_model * elem, rows * d_ffn * elem
    launches = {
        # name: (FLOPs, bytes read + written)
        "dispatch+gemm1": (2.0 * g * rows * d_model * d_ffn, x + w1 + h * (1 + g)),          # h_act + pre-activations
        "gemm2+combine": (2.0 * rows * d_model * d_ffn, h + w2 + x),
        "dy dispatch+dgrad2": (2.0 * rows * d_model * d_ffn, x + w2 + h * g + h * g),         # reads pre-activations, writes dh(,dh2)
        "wgrad2": (2.0 * rows * d_model * d_ffn, x + h + w2),
        "wgrad1": (2.0 * g * rows * d_model * d_ffn, h * g + x * g + w1),
        "dgrad1+combine": (2.0 * g * rows * d_model * d_ffn, h * g + w1 + x),
    }
    out = {}
    for name, (fl, by) in launches.items():
        t_c, t_m = fl / (peak_tflops * 1e9), by / (hbm_gbs * 1e6)
        out[name] = {"ms": round(max(t_c, t_m), 4), "compute_ms": round(t_c, 4), "hbm_ms": round(t_m, 4),
                     "bound": "compute" if t_c >= t_m else "hbm", "expected_tensor_pct": round(100 * t_c / max(t_c, t_m), 1),
                     "expected_dram_pct": round(100 * t_m / max(t_c, t_m), 1)}
    out["total_ms"] = round(sum(v["ms"] for v in out.values()), 4)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--d-model", type=int, default=4096)
    ap.add_argument("--d-ffn", type=int, default=14336)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--act", default="swiglu")
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--forward-only", action="store_true")
    ap.add_argument("--kept-fraction", type=float, default=1.0)
    ap.add_argument("--measured-ms", type=float, default=0.0)
    ap.add_argument("--experts-per-gpu", type=int, default=0, help="include the HBM traffic of this many experts' weights")
    ap.add_argument("--per-kernel", action="store_true",
                    help="print the expected duration and bound of each GEMM launch instead (needs --experts-per-gpu)")
    a = ap.parse_args()
    if a.per_kernel:
        rows = int(a.tokens * a.top_k * a.kept_fraction)
        print(json.dumps(kernel_estimates(rows, a.d_model, a.d_ffn, max(1, a.experts_per_gpu), a.act), indent=1))
        return
    r = roofline(a.tokens, a.d_model, a.d_ffn, a.top_k, a.act, a.gpus, not a.forward_only, a.kept_fraction,
                 experts_per_gpu=a.experts_per_gpu)
    if a.measured_ms > 0:
        r["measured_ms"] = a.measured_ms
        r["fraction_of_roofline"] = round(r["target_ms"] / a.measured_ms, 3)
        # the same against the sustained (power-capped) GEMM rate, the ceiling that applies to a step-long kernel sequence
        sus = roofline(a.tokens, a.d_model, a.d_ffn, a.top_k, a.act, a.gpus, not a.forward_only, a.kept_fraction,
                       peak_tflops=measured_sustained_tflops(), experts_per_gpu=a.experts_per_gpu)
        r["sustained_peak_tflops"] = sus["peak_tflops"]
        r["fraction_of_roofline_sustained"] = round(sus["target_ms"] / a.measured_ms, 3)
    print(json.dumps(r))


if __name__ == "__main__":
    main()
