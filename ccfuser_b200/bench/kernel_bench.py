"""Fused kernels against NCCL all-to-all + library GEMM (the fig. 12 experiment of the reference:
mix_moe/mix_moe/kernel_evaluation.py:193-463 with the timing loops of mix_moe/csrc/cuda/mix_gemm.cu:619-662).

"AG" = dispatch all-to-all -> GEMM-1 (one fused kernel here), "GA" = GEMM-2 -> combine all-to-all (one fused kernel
plus the wait/reduce on the source). ``--ag-epilogue plain`` (default) times what the reference's AG_test times, GEMM-1
with its bias and one output (mix_moe/csrc/mix_moe.h:146-185); ``layer`` times the training layer's kernel, which also
applies GELU and stores the pre-activation, and gives the baseline the same extra work. Routing is synthetic with a
chosen locality (fraction of a rank's tokens that
stay on the rank), top-1, 16384 tokens per GPU, 1024 -> 4096 -> 1024, swept over the remote fraction or over
experts per GPU. Everything is timed on the device with CUDA events, max over ranks.

    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 -m ccfuser_b200.bench.kernel_bench \
        --sweep remote
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .. import MoEConfig, MoELayer
from .. import native as N
from ..utils.dist import init_distributed


def synthetic_routing(tokens, e_loc, world, rank, remote_frac, gen):
    """Expert id per token: local with probability 1 - remote_frac, else uniformly on the other ranks."""
    local = torch.rand(tokens, generator=gen, device="cuda") >= remote_frac
    e_local = torch.randint(0, e_loc, (tokens,), generator=gen, device="cuda") + rank * e_loc
    if world == 1:
        return e_local.int().view(-1, 1)
    other = torch.randint(0, world - 1, (tokens,), generator=gen, device="cuda")
    other = other + (other >= rank).long()
    e_remote = torch.randint(0, e_loc, (tokens,), generator=gen, device="cuda") + other * e_loc
    return torch.where(local, e_local, e_remote).int().view(-1, 1)


def timed(fn, iters, warmup, world):
    out = []
    for i in range(warmup + iters):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        if i >= warmup:
            out.append(s.elapsed_time(e))
    t = torch.tensor([sorted(out)[len(out) // 2]], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def run(args, world, rank, e_loc, remote_frac):
    d, f, tokens = args.d_model, args.d_ffn, args.tokens
    cfg = MoEConfig(d_model=d, d_ffn=f, num_experts=e_loc * world, top_k=1, capacity_factor=None, activation="gelu",
                    dtype=torch.bfloat16, ep_size=world, backend="fused", max_tokens=tokens, recv_factor=2.5)
    layer = MoELayer(cfg, device="cuda")
    with torch.no_grad():
        for p in layer.parameters():
            p.normal_(0, 0.02)
    fm = layer._fused_impl()
    ex = layer.experts
    gen = torch.Generator(device="cuda").manual_seed(17 + rank)
    x = torch.randn(tokens, d, device="cuda", dtype=torch.bfloat16, generator=gen)
    idx = synthetic_routing(tokens, e_loc, world, rank, remote_frac, gen)
    gate = torch.ones(tokens, 1, device="cuda", dtype=torch.float32)
    y = torch.empty(tokens, d, device="cuda", dtype=torch.bfloat16)

    # fused AG needs a completed plan; GA needs GEMM-1's output and ends with the source-side reduce so that the
    # completion counters stay in step. Each timed call therefore runs the whole forward, with one stage timed.
    def forward(time_stage):
        fm.stage_route_plan(idx, tokens)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        ev[0].record()
        if args.ag_epilogue == "plain":
            fm.stage_dispatch_gemm1(x, idx, gate, ex.htoh4.weight, ex.htoh4.bias, save_pre=False, act=N.ACT_NONE)
        else:
            fm.stage_dispatch_gemm1(x, idx, gate, ex.htoh4.weight, ex.htoh4.bias)
        ev[1].record()
        fm.stage_gemm2_combine(ex.h4toh.weight, ex.h4toh.bias)
        fm.stage_reduce(tokens, y)
        ev[2].record()
        return ev

    ag, ga = [], []
    for i in range(args.warmup + args.iters):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ev = forward(None)
        torch.cuda.synchronize()
        if i >= args.warmup:
            ag.append(ev[0].elapsed_time(ev[1]))
            ga.append(ev[1].elapsed_time(ev[2]))
    fm.ctx.check_status("kernel bench")
    med = lambda v: sorted(v)[len(v) // 2]
    t = torch.tensor([med(ag), med(ga)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    fused_ag, fused_ga = float(t[0]), float(t[1])

    # ---- baseline: all_to_all_single + per-expert library GEMM ------------------------------------------------
    from ..ops.routing import route_local
    plan = route_local(idx.long(), cfg.num_experts, tokens)
    order = torch.sort(plan.expert, stable=True).indices
    send = x[order].contiguous()
    table = plan.count.clone()
    if world > 1:
        tl = [torch.empty_like(table) for _ in range(world)]
        dist.all_gather(tl, table)
        table = torch.stack(tl)
    else:
        table = table.view(1, -1)
    send_per = plan.count.view(world, e_loc).sum(1).tolist()
    recv_cnt = table[:, rank * e_loc:(rank + 1) * e_loc]
    recv_per = recv_cnt.sum(1).tolist()
    recv = torch.empty(sum(recv_per), d, device="cuda", dtype=torch.bfloat16)
    w1t = ex.htoh4.weight.detach()
    w2t = ex.h4toh.weight.detach()
    per_expert = recv_cnt.sum(0).tolist()
    h = torch.empty(sum(recv_per), f, device="cuda", dtype=torch.bfloat16)
    o = torch.empty(sum(recv_per), d, device="cuda", dtype=torch.bfloat16)
    back = torch.empty(tokens, d, device="cuda", dtype=torch.bfloat16)

    def a2a_in():
        if world > 1:
            dist.all_to_all_single(recv, send, recv_per, send_per)
        else:
            recv.copy_(send)

    b1t = ex.htoh4.bias.detach()
    layer_epi = args.ag_epilogue == "layer"
    pre = torch.empty_like(h) if layer_epi else None

    def gemm1():
        # rows arrive grouped by (source, expert); a real layer regroups them, here each segment is multiplied in place
        off = 0
        for r in range(world):
            for e in range(e_loc):
                c = int(recv_cnt[r, e])
                if c:
                    if layer_epi:
                        torch.addmm(b1t[e], recv[off:off + c], w1t[e].t(), out=pre[off:off + c])
                    else:
                        torch.addmm(b1t[e], recv[off:off + c], w1t[e].t(), out=h[off:off + c])
                off += c
        if layer_epi:
            h.copy_(torch.nn.functional.gelu(pre))

    def gemm2():
        off = 0
        for r in range(world):
            for e in range(e_loc):
                c = int(recv_cnt[r, e])
                if c:
                    torch.mm(h[off:off + c], w2t[e].t(), out=o[off:off + c])
                off += c

    def a2a_out():
        if world > 1:
            dist.all_to_all_single(back, o, send_per, recv_per)
        else:
            back.copy_(o)

    # stronger baseline: regroup the received rows to expert-major and use the library grouped GEMM
    seg = recv_cnt.reshape(-1).tolist()
    starts = [0]
    for c in seg:
        starts.append(starts[-1] + c)
    perm = torch.cat([torch.arange(starts[r * e_loc + e], starts[r * e_loc + e + 1]) for e in range(e_loc) for r in range(world)]
                     + [torch.zeros(0, dtype=torch.long)]).to("cuda")
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel(), device="cuda")
    offs = torch.tensor(per_expert, device="cuda", dtype=torch.int32).cumsum(0).to(torch.int32)
    has_grouped = hasattr(torch, "_grouped_mm")

    eid = torch.repeat_interleave(torch.arange(e_loc, device="cuda"), torch.tensor(per_expert, device="cuda"))

    def gemm1_grouped():
        z = torch._grouped_mm(recv.index_select(0, perm), w1t.transpose(1, 2), offs=offs) + b1t[eid]
        return torch.nn.functional.gelu(z) if layer_epi else z

    hg = gemm1_grouped() if has_grouped else None

    def gemm2_grouped():
        o.copy_(torch._grouped_mm(hg, w2t.transpose(1, 2), offs=offs).index_select(0, inv))

    base_a2a_in = timed(a2a_in, args.iters, args.warmup, world)
    base_ag = timed(lambda: (a2a_in(), gemm1()), args.iters, args.warmup, world)
    base_a2a_out = timed(a2a_out, args.iters, args.warmup, world)
    base_ga = timed(lambda: (gemm2(), a2a_out()), args.iters, args.warmup, world)
    grouped_ag = timed(lambda: (a2a_in(), gemm1_grouped()), args.iters, args.warmup, world) if has_grouped else None
    grouped_ga = timed(lambda: (gemm2_grouped(), a2a_out()), args.iters, args.warmup, world) if has_grouped else None
    layer.release()
    del layer
    torch.cuda.empty_cache()
    return {"bench": "fused_kernels_vs_nccl", "ag_epilogue": args.ag_epilogue, "n_gpus": world, "tokens_per_gpu": tokens, "d_model": d, "d_ffn": f,
            "experts_per_gpu": e_loc, "remote_frac": remote_frac,
            "fused_ag_ms": round(fused_ag, 4), "nccl_a2a_gemm1_ms": round(base_ag, 4), "nccl_a2a_in_ms": round(base_a2a_in, 4),
            "fused_ga_ms": round(fused_ga, 4), "gemm2_nccl_a2a_ms": round(base_ga, 4), "nccl_a2a_out_ms": round(base_a2a_out, 4),
            "nccl_a2a_grouped_gemm1_ms": None if grouped_ag is None else round(grouped_ag, 4),
            "grouped_gemm2_nccl_a2a_ms": None if grouped_ga is None else round(grouped_ga, 4),
            "ag_speedup": round(base_ag / fused_ag, 2), "ga_speedup": round(base_ga / fused_ga, 2),
            "ag_speedup_vs_grouped": None if grouped_ag is None else round(grouped_ag / fused_ag, 2),
            "ga_speedup_vs_grouped": None if grouped_ga is None else round(grouped_ga / fused_ga, 2)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sweep", default="remote", choices=["remote", "experts", "single"])
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--d-model", type=int, default=1024)
    ap.add_argument("--d-ffn", type=int, default=4096)
    ap.add_argument("--experts-per-gpu", type=int, default=16)
    ap.add_argument("--remote-frac", type=float, default=0.25)
    ap.add_argument("--ag-epilogue", default="plain", choices=["plain", "layer"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rank, _, world = init_distributed()
    if args.sweep == "remote":
        # the reference sweeps the locality 0.55, 0.60, ... 1.0 (mix_moe/mix_moe/kernel_evaluation.py:366-369)
        grid = [(args.experts_per_gpu, round(0.45 - 0.05 * i, 2)) for i in range(10)]
    elif args.sweep == "experts":
        grid = [(e, args.remote_frac) for e in (2, 4, 8, 16, 32, 64)]
    else:
        grid = [(args.experts_per_gpu, args.remote_frac)]
    if world == 1:
        grid = [(e, 0.0) for e, _ in grid]
        grid = list(dict.fromkeys(grid))
    results = []
    for e_loc, rf in grid:
        r = run(args, world, rank, e_loc, rf)
        results.append(r)
        if rank == 0:
            print(json.dumps(r), flush=True)
    if rank == 0 and args.out:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "w") as fh:
            for r in results:
                fh.write(json.dumps(r) + "\n")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
