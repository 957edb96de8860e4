"""Per-tile clock trace of the fused dispatch + GEMM-1 kernel on one GPU: when did each CTA pair finish pushing rows,
when did the operands of its first tile land, when did its first MMAs and its first epilogue finish. Shows that the tensor
cores start before the row push has ended (D / F environment variables select d_model / d_ffn).

    python -m ccfuser_b200.bench.overlap_trace
"""
import os

import torch

from .. import MoEConfig, MoELayer
from .kernel_bench import synthetic_routing

d, f, tokens, e_loc = int(os.environ.get("D", 2048)), int(os.environ.get("F", 8192)), 16384, 8
cfg = MoEConfig(d_model=d, d_ffn=f, num_experts=e_loc, top_k=1, activation="gelu", dtype=torch.bfloat16, ep_size=1, backend="fused", max_tokens=tokens, recv_factor=2.5)
layer = MoELayer(cfg, device="cuda"); fm = layer._fused_impl(); ex = layer.experts
gen = torch.Generator(device="cuda").manual_seed(1)
x = torch.randn(tokens, d, device="cuda", dtype=torch.bfloat16, generator=gen)
idx = synthetic_routing(tokens, e_loc, 1, 0, 0.0, gen)
gate = torch.ones(tokens, 1, device="cuda"); y = torch.empty(tokens, d, device="cuda", dtype=torch.bfloat16)
NT = 48
def fwd(tr1=None):
    fm.stage_route_plan(idx, tokens)
    fm.stage_dispatch_gemm1(x, idx, gate, ex.htoh4.weight, ex.htoh4.bias, trace=tr1)
    fm.stage_gemm2_combine(ex.h4toh.weight, ex.h4toh.bias)
    fm.stage_reduce(tokens, y)
for _ in range(3): fwd()
t1 = torch.zeros(148, NT, 8, dtype=torch.int64, device="cuda")
fwd(t1); torch.cuda.synchronize()
t = t1.cpu().double()
lead = t[0::2]     # leader CTAs of the pairs record the MMA events
start = lead[:, NT-1, 0]; disp = lead[:, NT-1, 1]
first_ops = lead[:, 0, 4]; first_commit = lead[:, 0, 5]; first_epi = lead[:, 0, 7]
ntile = (lead[:, :NT-1, 7] > 0).sum(1)
last = torch.stack([lead[c, int(ntile[c])-1, 7] for c in range(lead.shape[0])])
ok = first_ops > 0
print(f"d={d} f={f}: per leader CTA, clocks after kernel start (median over {int(ok.sum())} CTAs):")
print(f"  this CTA's epilogue warps finished pushing rows : {float((disp-start)[ok].median()):.0f}")
print(f"  first operands of its first tile landed         : {float((first_ops-start)[ok].median()):.0f}")
print(f"  last MMA of its first tile committed            : {float((first_commit-start)[ok].median()):.0f}")
print(f"  first epilogue finished                         : {float((first_epi-start)[ok].median()):.0f}")
print(f"  kernel end (last epilogue)                      : {float((last-start)[ok].median()):.0f}")
print(f"  CTAs whose first MMA ran before their own push ended: {int(((first_ops < disp) & ok).sum())} of {int(ok.sum())}")
