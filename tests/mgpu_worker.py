"""Multi-GPU check of the fused layer, run as `torchrun --nproc-per-node W tests/mgpu_worker.py`.

Every rank builds the same full parameter set from a seed, keeps its expert shard, runs the fused forward and
backward several times, and compares with the dense fp32 oracle evaluated on the gathered inputs of all ranks
using the routing decisions of the kernels. Prints 'MGPU_OK' on rank 0 when everything matches.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ccfuser_b200 import MoEConfig, MoELayer  # noqa: E402
from ccfuser_b200.ops.fused import _FusedMoEFn, topk_softmax  # noqa: E402
from ccfuser_b200.ops.reference import dense_moe_oracle  # noqa: E402
from ccfuser_b200.utils.dist import init_distributed  # noqa: E402


def rel(a, b):
    """Relative Frobenius error. (A max-norm check is too sharp for ReLU: a pre-activation whose sign differs
    between the bf16 kernel and the fp32 oracle flips one gradient element completely.)"""
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm().clamp_min(1e-6))


def gather(t, world):
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t.contiguous())
    return out


def run_case(rank, world, act, cf, tokens, e_loc, d, f, iters=3):
    torch.manual_seed(7)
    e = e_loc * world
    cfg = MoEConfig(d_model=d, d_ffn=f, num_experts=e, top_k=2, capacity_factor=cf, activation=act,
                    dtype=torch.bfloat16, ep_size=world, backend="fused", max_tokens=tokens)
    layer = MoELayer(cfg, device="cuda")
    names = ["htoh4", "h4toh"] + (["htoh4_gate"] if act == "swiglu" else [])
    full = {}
    g = torch.Generator(device="cuda").manual_seed(11)
    full["gate.weight"] = (torch.randn(e, d, device="cuda", generator=g) * 0.05).bfloat16()
    for n in names:
        shp = getattr(layer.experts, n).weight.shape[1:]
        full[n + ".weight"] = (torch.randn(e, *shp, device="cuda", generator=g) * 0.05).bfloat16()
        full[n + ".bias"] = (torch.randn(e, shp[0], device="cuda", generator=g) * 0.05).bfloat16()
    sl = slice(rank * e_loc, (rank + 1) * e_loc)
    with torch.no_grad():
        layer.gate.gate.weight.copy_(full["gate.weight"])
        layer.gate.gate.bias.zero_()
        for n in names:
            getattr(layer.experts, n).weight.copy_(full[n + ".weight"][sl])
            getattr(layer.experts, n).bias.copy_(full[n + ".bias"][sl])
    fm = layer._fused_impl()
    ex = layer.experts
    worst = 0.0
    for it in range(iters):
        gx = torch.Generator(device="cuda").manual_seed(100 * it + rank)
        # uneven token counts across ranks exercise ragged segments
        t_r = tokens - 37 * rank - 5 * it
        x = (torch.randn(t_r, d, device="cuda", generator=gx) * 0.5).bfloat16().requires_grad_(True)
        idx, w = topk_softmax(layer.gate.logits(x.detach()), 2)
        w = w.detach().requires_grad_(True)
        for p in layer.parameters():
            p.grad = None
        wg = ex.htoh4_gate.weight if act == "swiglu" else None
        bg = ex.htoh4_gate.bias if act == "swiglu" else None
        y = _FusedMoEFn.apply(x, w, idx, ex.htoh4.weight, ex.htoh4.bias, wg, bg, ex.h4toh.weight, ex.h4toh.bias, fm)
        gy = torch.randn(t_r, d, device="cuda", generator=gx).bfloat16()
        y.backward(gy)
        torch.cuda.synchronize()
        fm.ctx.check_status(f"{act} it{it}")
        # oracle on all ranks' data (token counts differ: pad to `tokens` rows for the gather, then cut)
        def padded(t, fill=0):
            out = torch.full((tokens,) + tuple(t.shape[1:]), fill, dtype=t.dtype, device=t.device)
            out[:t.shape[0]] = t
            return out
        counts = [int(c) for c in gather(torch.tensor([t_r], device="cuda"), world)]
        xs = [a[:c] for a, c in zip(gather(padded(x.detach()), world), counts)]
        idxs = [a[:c] for a, c in zip(gather(padded(idx), world), counts)]
        ws = [a[:c] for a, c in zip(gather(padded(w.detach()), world), counts)]
        gys = [a[:c] for a, c in zip(gather(padded(gy), world), counts)]
        fp = {k: v.float().requires_grad_(k != "gate.weight") for k, v in full.items()}
        xf = [a.float().requires_grad_(True) for a in xs]
        wf = [a.float().requires_grad_(True) for a in ws]
        ys = []
        for r in range(world):
            cap = cfg.capacity(counts[r])
            ys.append(dense_moe_oracle([xf[r]], fp, top_k=2, capacity=cap, activation=act, routing=[(idxs[r], wf[r])])[0])
        sum((a * b.float()).sum() for a, b in zip(ys, gys)).backward()
        errs = {"y": rel(y, ys[rank]), "dx": rel(x.grad, xf[rank].grad), "dw_gate": rel(w.grad, wf[rank].grad)}
        for n in names:
            errs["d" + n + ".w"] = rel(getattr(ex, n).weight.grad, fp[n + ".weight"].grad[sl])
            errs["d" + n + ".b"] = rel(getattr(ex, n).bias.grad, fp[n + ".bias"].grad[sl])
        bad = {k: v for k, v in errs.items() if not v < 3e-2}
        if bad:
            raise AssertionError(f"rank {rank} {act} cf={cf} it={it}: {bad}")
        worst = max(worst, max(errs.values()))
    return worst


def main():
    rank, local_rank, world = init_distributed()
    cases = [("gelu", 1.25, 1024, 4, 256, 512), ("swiglu", None, 700, 2, 256, 384), ("relu", 1.0, 2048, 8, 512, 1024)]
    worst = 0.0
    for act, cf, tokens, e_loc, d, f in cases:
        worst = max(worst, run_case(rank, world, act, cf, tokens, e_loc, d, f))
        dist.barrier()
    t = torch.tensor([worst], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(f"MGPU_OK world={world} worst_rel_err={float(t):.4f}", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
