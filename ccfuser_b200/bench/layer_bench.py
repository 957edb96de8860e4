"""MoE layer forward+backward benchmark (the fig. 10 measurement of the reference,
mix_moe/mix_moe/examples/mix_moe_ddp.py:155-210 and mix_moe/mix_moe/test.py:17-137), device-timed with CUDA
events, max over ranks, for the fused backend or the NCCL all-to-all + library GEMM baseline.

    python -m ccfuser_b200.bench.layer_bench --tokens 16384 --d-model 4096 --d-ffn 14336 --experts-per-gpu 8 \
        --act swiglu --cf 1.2
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m ccfuser_b200.bench.layer_bench ...

One JSON line per configuration: forward / backward / total ms, achieved TFLOP/s per GPU, and the roofline
fraction = max(FLOPs / measured GEMM peak, NVLink bytes / link bandwidth) / measured time.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .. import MoEConfig, MoELayer, zipf_router_bias
from ..utils.dist import init_distributed
from .gemm_bench import measured_peaks, measured_sustained_tflops

NVLINK_GBS = 770.0  # measured peer-copy bandwidth per direction per GPU on this pool (900 nominal)


def run_config(args, world, rank, tokens, experts_per_gpu, backend):
    dtype = torch.float16 if args.dtype == "fp16" else torch.bfloat16
    cfg = MoEConfig(d_model=args.d_model, d_ffn=args.d_ffn, num_experts=experts_per_gpu * world, top_k=args.top_k,
                    capacity_factor=args.cf if args.cf > 0 else None, activation=args.act, bias=not args.no_bias,
                    dtype=dtype, ep_size=world, backend=backend, max_tokens=tokens, recv_factor=args.recv_factor,
                    shadow_experts=args.shadow)
    layer = MoELayer(cfg, device="cuda")
    with torch.no_grad():
        for p in layer.parameters():
            p.normal_(0, 0.02)
        if args.zipf > 0:
            layer.gate.gate.bias.copy_(zipf_router_bias(cfg.num_experts, args.zipf, args.zipf_scale).to(dtype))
    g = torch.Generator(device="cuda").manual_seed(1 + rank)
    x = torch.randn(tokens, args.d_model, device="cuda", dtype=dtype, generator=g).requires_grad_(not args.forward_only)
    gy = torch.randn(tokens, args.d_model, device="cuda", dtype=dtype, generator=g)
    flush = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    fwd, bwd = [], []
    moved = None
    graphed = None
    if args.graph and args.forward_only and backend == "fused":
        from ..ops.fused import GraphedForward
        graphed = GraphedForward(layer, tokens)
    for it in range(args.warmup + args.iters):
        for p in layer.parameters():
            p.grad = None
        x.grad = None
        flush.zero_()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        if graphed is not None:
            y = graphed(x)
            e1.record()
            e2.record()
        elif args.forward_only:
            with torch.no_grad():
                y = layer(x)
            e1.record()
            e2.record()
        else:
            y = layer(x)
            e1.record()
            y.backward(gy)
            e2.record()
        torch.cuda.synchronize()
        if it >= args.warmup:
            fwd.append(e0.elapsed_time(e1))
            bwd.append(e1.elapsed_time(e2))
        elif args.rebalance and it == max(0, args.warmup - 2) and world > 1 and graphed is None:
            # one re-placement from the counts of this warm-up call; the remaining warm-up call runs on the new layout
            pl = layer.rebalance()
            moved = sum(1 for slot, old in enumerate(pl) if slot // experts_per_gpu != old // experts_per_gpu)
    if backend == "fused":
        layer._fused_impl().ctx.check_status("layer bench")
    med = lambda v: sorted(v)[len(v) // 2]
    t = torch.tensor([med(fwd), med(bwd), med([a + b for a, b in zip(fwd, bwd)])], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    stats = {}
    if backend == "fused":
        fm = layer._fused_impl()
        table = fm.table_copy.cpu()
        kept = int(table[rank].sum())
        stats = {"kept_rows_this_rank": kept, "dropped_frac": round(1 - kept / (tokens * args.top_k), 4),
                 "recv_rows_this_rank": int(fm.group_rows.sum().item()),
                 "remote_frac": round(1 - float(table[rank, rank * experts_per_gpu:(rank + 1) * experts_per_gpu].sum()) / max(1, kept), 4)}
    mats = 3 if args.act == "swiglu" else 2
    rows = tokens * args.top_k
    if backend == "fused":
        # rows this rank's experts actually processed (dropped slots do no work); max over ranks like the time
        rr = torch.tensor([float(stats["recv_rows_this_rank"])], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(rr, op=dist.ReduceOp.MAX)
        rows = int(rr.item())
        stats["max_recv_rows_over_ranks"] = rows
    flops_fwd = 2.0 * mats * args.d_model * args.d_ffn * rows
    flops = flops_fwd * (1 if args.forward_only else 3)
    peak, _, src = measured_peaks()
    total_ms = float(t[2]) if not args.forward_only else float(t[0])
    nv_bytes = rows * args.d_model * 2 * (world - 1) / max(1, world) * (2 if args.forward_only else 4)
    roof_ms = max(flops / (peak * 1e9), nv_bytes / (NVLINK_GBS * 1e6))
    roof_sus_ms = max(flops / (measured_sustained_tflops() * 1e9), nv_bytes / (NVLINK_GBS * 1e6))
    out = {"bench": "moe_layer", "backend": backend, "n_gpus": world, "tokens_per_gpu": tokens, "d_model": args.d_model,
           "d_ffn": args.d_ffn, "experts_per_gpu": experts_per_gpu, "top_k": args.top_k, "act": args.act, "cf": args.cf,
           "zipf": args.zipf, "shadow_experts": args.shadow, "dtype": args.dtype, "cuda_graph": graphed is not None, "experts_moved_by_rebalance": moved, "fwd_ms": round(float(t[0]), 4), "bwd_ms": round(float(t[1]), 4),
           "total_ms": round(total_ms, 4), "tflops_per_gpu": round(flops / total_ms / 1e9, 1),
           "nvlink_bytes_per_gpu": int(nv_bytes), "roofline_ms": round(roof_ms, 4),
           "roofline_frac_of_" + src: round(roof_ms / total_ms, 3),
           "roofline_frac_of_" + src + "_sustained": round(roof_sus_ms / total_ms, 3), **stats}
    layer.release()
    del layer
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="16384", help="tokens per GPU; comma list to sweep")
    ap.add_argument("--d-model", type=int, default=4096)
    ap.add_argument("--d-ffn", type=int, default=14336)
    ap.add_argument("--experts-per-gpu", default="8", help="comma list to sweep")
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--act", default="swiglu")
    ap.add_argument("--cf", type=float, default=1.2, help="capacity factor; 0 = no dropping")
    ap.add_argument("--recv-factor", type=float, default=2.0)
    ap.add_argument("--no-bias", action="store_true")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--zipf", type=float, default=0.0, help="Zipf exponent of expert popularity (router bias); 0 = off")
    ap.add_argument("--zipf-scale", type=float, default=1.0)
    ap.add_argument("--rebalance", action="store_true", help="re-place the experts once during the warm-up (needs --warmup >= 2)")
    ap.add_argument("--shadow", type=int, default=0, help="replicate the n most popular experts of every step on all ranks")
    ap.add_argument("--backends", default="fused", help="comma list of fused,nccl")
    ap.add_argument("--forward-only", action="store_true")
    ap.add_argument("--graph", action="store_true", help="with --forward-only: replay the fused forward from a CUDA graph")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rank, _, world = init_distributed()
    results = []
    for tokens in [int(v) for v in args.tokens.split(",")]:
        for epg in [int(v) for v in args.experts_per_gpu.split(",")]:
            for backend in args.backends.split(","):
                r = run_config(args, world, rank, tokens, epg, backend)
                results.append(r)
                if rank == 0:
                    print(json.dumps(r), flush=True)
    if rank == 0 and args.out:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "w") as f:
            for r in results:
                f.write(json.dumps(r) + "\n")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
