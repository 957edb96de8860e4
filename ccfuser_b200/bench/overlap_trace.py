"""Per-tile clock trace of the fused dispatch + GEMM-1 kernel on one GPU: when did each CTA pair finish pushing rows,
when did the operands of its first tile land, when did its first MMAs and its first epilogue finish; and, per tile, how
long the main loop took against its ideal, how long the MMA warp waited for a free accumulator and how long the
epilogue took. Shows that the tensor cores start before the row push has ended.

    python -m ccfuser_b200.bench.overlap_trace                 # d_model 2048, d_ffn 8192
    D=1024 F=4096 python -m ccfuser_b200.bench.overlap_trace
    D=4096 F=14336 TOKENS=256 E_LOC=1 ACT=swiglu python -m ccfuser_b200.bench.overlap_trace   # the small-message shape

Trace layout (``trace=`` of ops/gemm.py:launch): int64 ``[CTA, tile slot, 8]`` SM clock stamps {0 tile fetched, 1 rows
arrived, 2 last load issued, 3 accumulator free, 4 first operands landed, 5 last MMA committed, 6 accumulator full,
7 epilogue done}; the last slot of every CTA holds {0: kernel start, 1: this CTA's dispatch part finished}.
"""
from __future__ import annotations

import os
from typing import Dict

import torch

TENSOR_CYCLES_PER_KBLOCK = 512      # one 64-deep k-block of a 128 x 256 tile (or of a 256 x 256 pair tile on two SMs)


def analyze(trace: torch.Tensor, kblocks: int, leaders_only: bool = True) -> Dict[str, float]:
    """Medians over all recorded tiles, in SM clocks: main-loop time and its ratio to the tensor-pipe ideal, the MMA
    warp's wait for a free accumulator (epilogue not keeping up), the producer's wait for rows, epilogue time."""
    t = trace.detach().cpu().double()
    if leaders_only:
        t = t[0::2]                              # in the CTA-pair kernel the leader records the MMA events
    tiles = t[:, :-1]
    done = tiles[..., 7] > 0
    if not bool(done.any()):
        return {"tiles": 0}
    main = (tiles[..., 5] - tiles[..., 4])[done]
    epi = (tiles[..., 7] - tiles[..., 6])[done]
    rows_wait = (tiles[..., 1] - tiles[..., 0])[done]
    # accumulator wait of tile i = its 'accumulator free' stamp minus the previous tile's 'last MMA committed'
    prev_commit = torch.cat([t[:, -1:, 0], tiles[:, :-1, 5]], dim=1)
    acc_wait = (tiles[..., 3] - prev_commit)[done].clamp_min(0)
    ideal = kblocks * TENSOR_CYCLES_PER_KBLOCK
    med = lambda v: float(v.median())            # noqa: E731
    return {"tiles": int(done.sum()), "main_loop_clk": med(main), "main_loop_ideal_clk": float(ideal),
            "main_loop_efficiency": round(ideal / max(1.0, med(main)), 3), "acc_wait_clk": med(acc_wait),
            "rows_wait_clk": med(rows_wait), "epilogue_clk": med(epi)}


def main():
    from .. import MoEConfig, MoELayer
    from .kernel_bench import synthetic_routing
    d, f = int(os.environ.get("D", 2048)), int(os.environ.get("F", 8192))
    tokens, e_loc, act = int(os.environ.get("TOKENS", 16384)), int(os.environ.get("E_LOC", 8)), os.environ.get("ACT", "gelu")
    cfg = MoEConfig(d_model=d, d_ffn=f, num_experts=e_loc, top_k=1, activation=act, bias=act != "swiglu", dtype=torch.bfloat16, ep_size=1,
                    backend="fused", max_tokens=tokens, recv_factor=2.5)
    layer = MoELayer(cfg, device="cuda")
    fm, ex = layer._fused_impl(), layer.experts
    gen = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(tokens, d, device="cuda", dtype=torch.bfloat16, generator=gen)
    idx = synthetic_routing(tokens, e_loc, 1, 0, 0.0, gen)
    gate = torch.ones(tokens, 1, device="cuda")
    y = torch.empty(tokens, d, device="cuda", dtype=torch.bfloat16)
    nt = 48

    def fwd(tr1=None):
        fm.stage_route_plan(idx, tokens)
        swiglu = act == "swiglu"
        fm.stage_dispatch_gemm1(x, idx, gate, ex.htoh4.weight, ex.htoh4.bias, ex.htoh4_gate.weight if swiglu else None,
                                ex.htoh4_gate.bias if swiglu else None, trace=tr1, save_pre=False)
        fm.stage_gemm2_combine(ex.h4toh.weight, ex.h4toh.bias)
        fm.stage_reduce(tokens, y)

    for _ in range(3):
        fwd()
    t1 = torch.zeros(148, nt, 8, dtype=torch.int64, device="cuda")
    fwd(t1)
    torch.cuda.synchronize()
    t = t1.cpu().double()
    pair = fm._call_two_cta is not False
    lead = t[0::2] if pair else t     # in the CTA-pair kernel the leader CTAs record the MMA events
    start, disp = lead[:, nt - 1, 0], lead[:, nt - 1, 1]
    first_ops, first_commit, first_epi = lead[:, 0, 4], lead[:, 0, 5], lead[:, 0, 7]
    ntile = (lead[:, :nt - 1, 7] > 0).sum(1)
    last = torch.stack([lead[c, int(ntile[c]) - 1, 7] for c in range(lead.shape[0])])
    ok = first_ops > 0
    print(f"d={d} f={f}: per leader CTA, clocks after kernel start (median over {int(ok.sum())} CTAs):")
    print(f"  this CTA's epilogue warps finished pushing rows : {float((disp - start)[ok].median()):.0f}")
    print(f"  first operands of its first tile landed         : {float((first_ops - start)[ok].median()):.0f}")
    print(f"  last MMA of its first tile committed            : {float((first_commit - start)[ok].median()):.0f}")
    print(f"  first epilogue finished                         : {float((first_epi - start)[ok].median()):.0f}")
    print(f"  kernel end (last epilogue)                      : {float((last - start)[ok].median()):.0f}")
    print(f"  CTAs whose first MMA ran before their own push ended: {int(((first_ops < disp) & ok).sum())} of {int(ok.sum())}")
    print("  per tile:", analyze(t1, kblocks=(d + 63) // 64, leaders_only=pair))


if __name__ == "__main__":
    main()
