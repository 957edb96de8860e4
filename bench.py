#!/usr/bin/env python
"""Headline benchmark: end-to-end GPT-MoE training step, tokens/s over all GPUs of one node.

Model: 24 layers, d_model 2048, 16 heads, seq 1024, vocab 50257, MoE FFN (64 experts, top-2,
2048 -> 8192 -> 2048, GELU) in every other layer, expert-parallel over all N GPUs, data-parallel for the
replicated parameters; bf16; SGD; synthetic uniform-random token ids, random-init weights.
Per GPU batch is fixed (weak scaling). One JSON line is printed by rank 0.

    python bench.py --gpus 1 --steps 8 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        bench.py --gpus 8 --steps 8 --warmup 3
    python bench.py --impl reference ...     # the unmodified reference, if it could be installed
"""
import argparse
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "nccl"])
    ap.add_argument("--batch", type=int, default=8, help="sequences per GPU")
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--no-layer-bench", action="store_true")
    ap.add_argument("--rebalance", type=int, default=1,
                    help="1 (default): after the warm-up, every MoE layer moves experts between GPUs to the placement planned "
                         "from its observed routing counts, if that lowers the busiest GPU's load by at least 1 %% (same "
                         "model function; outside the timed region; needs more than one GPU). 0: keep the initial placement")
    ap.add_argument("--fuse-expert-sgd", type=int, default=1,
                    help="1 (default): the expert weights' SGD update runs in the epilogue of the weight-gradient GEMMs "
                         "(MoELayer.fuse_sgd: every expert matrix on one GPU, the second projection on 2 or more): the same "
                         "update, without writing those gradients and reading them and the weights again; measured 5 %% "
                         "faster per step with all 64 experts on one GPU. 0: separate optimizer pass for all parameters")
    ap.add_argument("--no-baseline", action="store_true",
                    help="skip the repository's own baseline arm (same model on the all_to_all_single + library "
                         "grouped-GEMM backend), against which vs_baseline is reported")
    ap.add_argument("--baseline-steps", type=int, default=4)
    ap.add_argument("--check", action="store_true",
                    help="before timing, check the fused layer's forward at the layer benchmark's shape against a sampled fp32 oracle")
    ap.add_argument("--breakdown", default="",
                    help="write a per-category table of one step's kernel time (torch.profiler, outside the timed region) "
                         "to this JSON file")
    return ap.parse_args()


def reference_arm(args):
    """The reference arm. The only install allowed for it did not produce a package (see
    baseline/INSTALL_RESULT.txt), so this prints the `unavailable` line and exits 0."""
    note = os.path.join(ROOT, "baseline", "INSTALL_RESULT.txt")
    why = "reference not installed"
    if os.path.exists(note):
        why = open(note).read().strip().splitlines()[0]
    if int(os.environ.get("RANK", 0)) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def layer_bench(torch, dist, world, rank, steps=5, warmup=3):
    """MoE layer fwd+bwd (d_model 4096, SwiGLU 4096->14336->4096, 8 experts per GPU, top-2, capacity 1.2,
    16384 tokens per GPU, bf16): device-timed ms, max over ranks."""
    from ccfuser_b200 import MoEConfig, MoELayer
    tokens = 16384
    cfg = MoEConfig(d_model=4096, d_ffn=14336, num_experts=8 * world, top_k=2, capacity_factor=1.2, activation="swiglu",
                    bias=False, dtype=torch.bfloat16, ep_size=world, backend="fused", max_tokens=tokens)
    layer = MoELayer(cfg, device="cuda")
    with torch.no_grad():
        for p in layer.parameters():
            p.normal_(0, 0.02)
    x = torch.randn(tokens, 4096, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    gy = torch.randn(tokens, 4096, device="cuda", dtype=torch.bfloat16)
    times = []
    for i in range(warmup + steps):
        for p in layer.parameters():
            p.grad = None
        x.grad = None
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        layer(x).backward(gy)
        e.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(s.elapsed_time(e))
    layer._fused_impl().ctx.check_status("layer bench")
    ms = sorted(times)[len(times) // 2]
    # rows the busiest rank's experts actually processed (slots beyond the capacity do no work), like the time: max over ranks
    rows = float(layer._fused_impl().group_rows.sum())
    t = torch.tensor([ms, rows], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, rows = float(t[0]), float(t[1])
    flops = 3 * 2 * 3 * 4096 * 14336 * rows  # (fwd + 2x bwd) x 2 FLOP x 3 matrices x processed rows
    layer.release()
    del layer
    torch.cuda.empty_cache()
    out = {"fwd_bwd_ms": round(ms, 3), "tflops_per_gpu": round(flops / ms / 1e9, 1), "rows_processed_max_rank": int(rows),
           "slots_per_rank": tokens * 2,
           "config": "16384 tok/GPU, d4096, SwiGLU ffn14336, 8 experts/GPU, top-2, cf1.2, bf16"}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
        out["frac_of_measured_cublas_burst"] = round(flops / ms / 1e9 / float(peaks["bf16_tflops"]), 3)
        out["frac_of_measured_cublas_sustained"] = round(flops / ms / 1e9 / float(peaks["bf16_tflops_sustained"]), 3)
    except Exception:
        pass
    return out


def release_model(torch, model):
    """Free a model's symmetric buffers (collective) and its memory before the next arm is built."""
    for m in model.moe_layers():
        m.release()
    torch.cuda.empty_cache()


def classify_kernel(kname: str, scopes: str, shapes: str, vocab_padded: int, d_ffn: int, tokens: int) -> str:
    """Category of one kernel of a training step, from its name and from the operator that launched it."""
    k = kname.lower()
    if "grouped_gemm" in k:
        return "moe_fused_gemms"
    if "combine_wait" in k:
        return "moe_wait_for_peers"
    if any(t in k for t in ("route_", "plan_kernel", "combine_reduce", "topk_softmax", "router_", "colsum_grouped", "dispatch_kernel")):
        return "moe_route_plan_reduce"
    if "sgd_step" in k or "sgd_multi" in k:
        return "optimizer"
    if "nccl" in k:
        return "nccl_allreduce"
    if any(t in k for t in ("flash", "fmha", "sdpa", "attention")) or "scaled_dot_product" in scopes:
        return "attention_core"
    if any(t in k for t in ("nvjet", "gemm", "cutlass", "xmma", "cublas")):
        if str(vocab_padded) in shapes:
            return "lm_head_gemms"
        # token count and FFN width coincide at the default size: the dense FFN is the GEMM with two such dimensions
        dims = shapes.replace("[", " ").replace("]", " ").replace(",", " ").split()
        if sum(1 for v in dims if v == str(d_ffn)) >= (2 if tokens == d_ffn else 1):
            return "dense_ffn_gemms"
        return "attention_projection_gemms"
    if any(t in scopes for t in ("cross_entropy", "log_softmax", "nll_loss")) or "softmax" in k:
        return "cross_entropy"
    if "layer_norm" in k or "layernorm" in scopes.lower():
        return "layernorm"
    return "elementwise_and_other"


def step_breakdown(torch, trainer, batch, c, tokens):
    """One training step under torch.profiler: kernel time per category in ms (this rank). Each kernel is taken once,
    from the operator that launched it."""
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA], record_shapes=True) as prof:
        trainer.step_device(*batch)
        torch.cuda.synchronize()
    table, names = {}, {}
    vocab_padded = (c.vocab_size + 127) // 128 * 128
    for ev in prof.events():
        kernels = getattr(ev, "kernels", None)
        if not kernels:
            continue
        scopes, node = [], ev
        while node is not None and len(scopes) < 12:
            scopes.append(node.name)
            node = getattr(node, "cpu_parent", None)
        scope_s, shape_s = " < ".join(scopes), str(getattr(ev, "input_shapes", ""))
        for kern in kernels:
            cat = classify_kernel(kern.name, scope_s, shape_s, vocab_padded, c.d_ffn, tokens)
            table[cat] = table.get(cat, 0.0) + kern.duration / 1e3
            key = (cat, kern.name[:60])
            names[key] = names.get(key, 0.0) + kern.duration / 1e3
    # kernels launched outside any recorded operator (library calls made through ctypes from plain Python code, e.g. the
    # optimizer) have no launching event: they are found as the difference, per kernel name, between all device events
    # and the attributed ones
    from torch.autograd import DeviceType
    seen, attributed = {}, {}
    cpu_names = {ev.name for ev in prof.events() if getattr(ev, "device_type", None) == DeviceType.CPU}
    for ev in prof.events():
        # device-side copies of host annotations (record_function ranges shown on the GPU timeline) are not kernels
        if (getattr(ev, "device_type", None) == DeviceType.CUDA and not getattr(ev, "is_async", False)
                and ev.name not in cpu_names):
            seen[ev.name] = seen.get(ev.name, 0.0) + float(getattr(ev, "device_time_total", 0.0) or 0.0) / 1e3
    for (cat, kname), v in list(names.items()):
        attributed[kname] = attributed.get(kname, 0.0) + v
    for kname_full, v in seen.items():
        kname = kname_full[:60]
        rest = v - attributed.get(kname, 0.0)
        if rest > 1e-3 and not kname_full.lower().startswith(("memcpy", "memset")):
            cat = classify_kernel(kname_full, "", "", vocab_padded, c.d_ffn, tokens)
            table[cat] = table.get(cat, 0.0) + rest
            names[(cat, kname)] = names.get((cat, kname), 0.0) + rest
            attributed[kname] = attributed.get(kname, 0.0) + rest
    total = sum(table.values())
    top = sorted(names.items(), key=lambda kv: -kv[1])[:25]
    return {"kernel_ms_by_category": {k: round(v, 3) for k, v in sorted(table.items(), key=lambda kv: -kv[1])},
            "kernel_ms_total": round(total, 3),
            "top_kernels": [{"category": k[0], "kernel": k[1], "ms": round(v, 3)} for k, v in top]}


def layer_check(torch, dist, world):
    """Sampled fp32 check of the fused layer's forward at the layer benchmark's shape (collective): 64 tokens per rank,
    every rank evaluating its own experts for all ranks' samples."""
    from ccfuser_b200 import MoEConfig, MoELayer
    from ccfuser_b200.ops.reference import sampled_oracle_check
    tokens = 16384
    cfg = MoEConfig(d_model=4096, d_ffn=14336, num_experts=8 * world, top_k=2, capacity_factor=1.2, activation="swiglu",
                    bias=False, dtype=torch.bfloat16, ep_size=world, backend="fused", max_tokens=tokens)
    layer = MoELayer(cfg, device="cuda")
    with torch.no_grad():
        for p in layer.parameters():
            p.normal_(0, 0.02)
        if world > 1:
            for p in layer.gate.parameters():
                dist.broadcast(p, 0)
        x = torch.randn(tokens, 4096, device="cuda", dtype=torch.bfloat16)
        fm = layer._fused_impl()
        idx, w = fm.route(x)
        y = fm.run_experts(x, idx, w)
        torch.cuda.synchronize()
        layer.check_status()
        err = sampled_oracle_check(layer, x, idx, w, y, n_sample=64, group=layer.ep_group if world > 1 else None)
    layer.release()
    del layer
    torch.cuda.empty_cache()
    t = torch.tensor([err["y"]], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {"forward_rel_err_sampled_max_over_ranks": round(float(t[0]), 5), "tolerance": 3e-2, "ok": bool(float(t[0]) < 3e-2)}


def run_arm(torch, dist, args, backend, steps, warmup, rank, local_rank, world, dev, batches, dev_batches, breakdown=False):
    """Build the model on one backend and time it: `steps` device-resident steps, then `steps` end-to-end steps (pinned
    host batch in, loss out). Returns this arm's record (times are max over ranks)."""
    from ccfuser_b200 import native as N
    from ccfuser_b200.models.gpt_moe import GPTMoE, GPTMoEConfig
    from ccfuser_b200.train import TrainStep
    from ccfuser_b200.utils.clocks import ClockSampler, visible_index
    seq = 1024
    torch.manual_seed(1234 + rank)       # both arms start from the same weights
    # no capacity factor (nothing is dropped, as in the reference); the receive buffers hold 4x the balanced load
    c = GPTMoEConfig(n_layer=args.layers, ep_size=world, backend=backend, max_tokens=args.batch * seq, seq_len=seq,
                     recv_factor=4.0)
    model = GPTMoE(c, device=dev)
    fused = backend == "fused"
    # optional on one GPU: the experts' SGD update inside the weight-gradient GEMMs (same update, no gradient round trip)
    fuse_sgd = fused and bool(args.fuse_expert_sgd)
    trainer = TrainStep(model, lr=1e-4, optimizer="sgd", fuse_expert_sgd=fuse_sgd)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def busiest_rank_load():
        loads = [float(m._fused.group_rows.sum()) for m in model.moe_layers() if m._fused is not None]
        t_l = torch.tensor([max(loads) if loads else 0.0], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t_l, op=dist.ReduceOp.MAX)
        return round(float(t_l) / (args.batch * seq * 2), 3)

    first_loss = None
    for i in range(warmup):
        l = trainer.step_device(*dev_batches[i % 4])
        if i == 0:
            first_loss = float(l)          # before any update: the same number on every backend up to rounding
    sync()
    moved = None
    imbalance_before = busiest_rank_load() if fused else None
    if args.rebalance and fused and world > 1:
        # expert placement from the routing counts of the last warm-up step, layer by layer (collective), then one
        # more untimed step so that the timed region starts from a steady state
        moved = 0
        e_loc = c.num_experts // world
        for m in model.moe_layers():
            # one NVSwitch node: a row that crosses GPUs costs next to nothing on the fused path, a rank above the mean
            # costs the whole group its excess, so the plan trades no balance for locality (slack 0)
            pl = m.rebalance(optimizer=trainer.opt, slack=0.0, min_gain=0.01)
            moved += sum(1 for slot, old in enumerate(pl) if slot // e_loc != old // e_loc)
        trainer.step_device(*dev_batches[0])
        sync()
    sampler = ClockSampler(visible_index(local_rank))
    sampler.start()
    launches0 = N.LAUNCHES[0]
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    s.record()
    for i in range(steps):
        loss = trainer.step_device(*dev_batches[i % 4])
    e.record()
    sync()
    ms = s.elapsed_time(e)
    launches = N.LAUNCHES[0] - launches0
    clocks = sampler.stop()
    # ---- end-to-end region: pinned host batch in, loss out, every step -----------------------------
    trainer.step(*batches[0])
    sync()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    last = 0.0
    for i in range(steps):
        last = trainer.step(*batches[i % 4])
    e2.record()
    sync()
    ms2 = s2.elapsed_time(e2)
    t = torch.tensor([ms, ms2], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    rec = {"backend": backend, "ms": float(t[0]), "ms_e2e": float(t[1]), "steps": steps, "launches": launches,
           "clocks": clocks, "first_loss": first_loss, "loss": float(loss.detach()), "last_loss": last, "moved": moved,
           "imbalance_before": imbalance_before, "imbalance": None, "overflow": None,
           "flops_per_token": c.flops_per_token(), "vocab": c.vocab_size, "fuse_sgd": fuse_sgd}
    if fused:
        from ccfuser_b200 import MoEOverflow
        for m in model.moe_layers():
            if m._fused is not None:
                try:
                    m._fused.ctx.check_status("bench")
                except MoEOverflow as ex:
                    rec["overflow"] = str(ex)
                break
        rec["imbalance"] = busiest_rank_load()
    if breakdown:
        rec["breakdown"] = step_breakdown(torch, trainer, dev_batches[0], c, args.batch * seq)
        sync()
    release_model(torch, model)
    del trainer, model
    torch.cuda.empty_cache()
    return rec


def main():
    args = parse()
    wd = float(os.environ.get("CCFUSER_BENCH_WATCHDOG_S", "0"))
    if wd > 0:
        # a stuck run prints every thread's Python stack and exits instead of waiting for an outer timeout
        import faulthandler
        faulthandler.dump_traceback_later(wd, exit=True)
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus > 1 and "RANK" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 400), os.path.abspath(__file__)] + sys.argv[1:]
        return subprocess.call(cmd)

    import torch
    import torch.distributed as dist
    from ccfuser_b200.utils.dist import init_distributed

    rank, local_rank, world = init_distributed()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    dev = torch.device("cuda", torch.cuda.current_device())
    seq = 1024
    tokens_per_step = args.batch * seq * world
    torch.manual_seed(99 + rank)

    def host_batch():
        ids = torch.randint(0, 50257, (args.batch, seq), dtype=torch.int64).pin_memory()
        return ids, ids.roll(-1, dims=1).contiguous().pin_memory()

    batches = [host_batch() for _ in range(4)]
    dev_batches = [(a.to(dev), b.to(dev)) for a, b in batches]
    check = None
    if args.check and args.impl == "ours":
        check = layer_check(torch, dist, world)
    main_backend = "fused" if args.impl == "ours" else "nccl"
    ours = run_arm(torch, dist, args, main_backend, args.steps, args.warmup, rank, local_rank, world, dev, batches,
                   dev_batches, breakdown=bool(args.breakdown))
    base = None
    if args.impl == "ours" and not args.no_baseline:
        try:
            base = run_arm(torch, dist, args, "nccl", max(1, args.baseline_steps), max(3, min(args.warmup, 3)), rank,
                           local_rank, world, dev, batches, dev_batches)
        except Exception as ex:     # the headline line survives a failure of the comparison arm
            base = {"error": repr(ex)[:300]}
    layer = None
    if not args.no_layer_bench and args.impl == "ours":
        try:
            layer = layer_bench(torch, dist, world, rank)
        except Exception as ex:  # keep the headline line even if the extra measurement fails
            layer = {"error": repr(ex)[:200]}
    if rank == 0:
        ms, ms2 = ours["ms"], ours["ms_e2e"]
        value = tokens_per_step * args.steps / (ms / 1e3)
        e2e_value = tokens_per_step * args.steps / (ms2 / 1e3)
        vs, own = None, None
        if base is not None and "error" not in base:
            b_value = tokens_per_step * base["steps"] / (base["ms"] / 1e3)
            b_e2e = tokens_per_step * base["steps"] / (base["ms_e2e"] / 1e3)
            vs = round(value / b_value, 3)
            own = {"what": "this repository's own baseline arm, NOT the reference: the same model, weights and batches on "
                           "torch all_to_all_single (NCCL) + library grouped GEMM (torch._grouped_mm) + torch activation; "
                           "one device-to-host read per layer call for the exchange sizes",
                   "value": round(b_value, 1), "unit": "tokens/s", "ms_per_step": round(base["ms"] / base["steps"], 3),
                   "e2e_value": round(b_e2e, 1), "steps": base["steps"], "e2e_ratio": round(e2e_value / b_e2e, 3),
                   "first_loss": base["first_loss"], "first_loss_abs_diff": abs(base["first_loss"] - ours["first_loss"]),
                   "clocks": base["clocks"]}
        elif base is not None:
            own = base
        out = {
            "metric": "gpt_moe_train_tokens_per_sec", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": vs,
            "vs_baseline_note": "value / own_baseline.value (the reference publishes no number for this metric and could "
                                "not be installed; see own_baseline.what)",
            "dtype": "bf16", "data": "synthetic", "impl": args.impl,
            "config": {"model": f"GPT-MoE {args.layers}L d2048 h16 seq1024 vocab50257, MoE every other layer (64 experts, top-2, ffn 8192, GELU)",
                       "global_batch": args.batch * world, "seq_len": seq, "parallelism": f"ep{world}" + (f"+dp{world}" if world > 1 else ""),
                       "optimizer": "sgd", "l2": "working set (weights + activations, tens of GB) far exceeds the 126 MB L2",
                       "loss": round(ours["loss"], 4), "first_loss": ours["first_loss"], "capacity_factor": None,
                       "mean_expert_grads": False,
                       "expert_sgd": (("applied in the weight-gradient GEMM epilogue (MoELayer.fuse_sgd)" if world == 1 else
                                       "second projection: in its weight-gradient GEMM's epilogue (MoELayer.fuse_sgd); first "
                                       "projection: separate optimizer pass") if ours.get("fuse_sgd")
                                      else "separate optimizer pass"),
                       "expert_placement": ("re-planned once from the routing counts of the last warm-up step, outside the "
                                            "timed region" if (args.rebalance and world > 1 and args.impl == "ours") else "initial"),
                       "max_rank_load_over_balanced": ours["imbalance"],
                       "max_rank_load_over_balanced_before_replacement": ours["imbalance_before"],
                       "overflow": ours["overflow"], "experts_moved_by_rebalance": ours["moved"]},
            "clocks": ours["clocks"],
            "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s",
                    "h2d_bytes_per_step": 2 * args.batch * seq * 8, "d2h_bytes_per_step": 4, "last_loss": round(ours["last_loss"], 4)},
            "gpu_launches": ours["launches"],
            "model_tflops_per_gpu": round(ours["flops_per_token"] * args.batch * seq / (ms / args.steps) / 1e9, 1),
        }
        if own is not None:
            out["own_baseline"] = own
        if layer is not None:
            out["moe_layer"] = layer
        if check is not None:
            out["check"] = check
        if args.breakdown and "breakdown" in ours:
            os.makedirs(os.path.dirname(os.path.abspath(args.breakdown)) or ".", exist_ok=True)
            with open(args.breakdown, "w") as f:
                json.dump({"n_gpus": world, "rank": 0, "ms_per_step_timed": round(ms / args.steps, 3),
                           "note": "kernel time of one step on rank 0 under torch.profiler, outside the timed region; kernels "
                                   "of concurrent streams (NCCL) overlap others, so the categories can add up to more than the step",
                           **ours["breakdown"]}, f, indent=1)
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
