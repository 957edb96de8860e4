"""Synthetic-data training loops for the three model families of the reference's end-to-end experiment
(GPT-2, BERT question answering, Transformer-XL; mix_moe/ae/fig11_data.sh, mix_moe/mix_moe/examples/models/
moe_gpt_ddp.py, moe_bert_ddp.py, mix_moe/mix_moe/examples/transformer-xl/train_ddp.py), each as a dense model, with
the NCCL all-to-all MoE baseline, or with the fused MoE layer.

    python -m ccfuser_b200.examples.train --model bert --variant fused --steps 20
    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 -m ccfuser_b200.examples.train \
        --model txl --variant fused

Prints ``STEP-i: step_time = ... ms`` lines and a ``[Summary] Average synchronized step_time`` line like the
reference scripts (mix_moe/mix_moe/examples/mix_moe_ddp.py:199,210), plus one JSON line with the same numbers.
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist
import torch.nn as nn

from ..models.bert_moe import BertMoEConfig, BertMoEForQuestionAnswering
from ..models.gpt_moe import GPTMoE, GPTMoEConfig
from ..models.transformer_xl_moe import TransformerXLMoE, TransformerXLMoEConfig
from ..parallel.ddp import wrap_ddp
from ..utils.dist import init_distributed


class _GPTStep(nn.Module):
    def __init__(self, m):
        super().__init__()
        self.m = m

    def forward(self, batch):
        return self.m(batch["ids"], batch["labels"])


class _BertStep(nn.Module):
    def __init__(self, m):
        super().__init__()
        self.m = m

    def forward(self, batch):
        return self.m(batch["ids"], batch["mask"], batch["types"], batch["start"], batch["end"])


class _TXLStep(nn.Module):
    def __init__(self, m):
        super().__init__()
        self.m = m
        self.mems = None

    def forward(self, batch):
        loss, self.mems = self.m(batch["ids"], batch["labels"], self.mems)
        return loss


def build(args, world, dev, ep_group=None):
    """``world`` is the size of the expert-parallel group (the whole job unless --ep-size says otherwise)."""
    backend = {"dense": "auto", "nccl": "nccl", "fused": "fused"}[args.variant]
    moe = args.variant != "dense"
    dtype = torch.float16 if args.dtype == "fp16" else torch.bfloat16
    g = torch.Generator().manual_seed(1 + (dist.get_rank() if dist.is_initialized() else 0))
    if args.model == "gpt":
        b, s = args.batch or 8, args.seq or 1024
        c = GPTMoEConfig(router_dtype=torch.float32 if args.router_fp32 else None, aux_loss_coef=args.aux_loss_coef,
                         z_loss_coef=args.z_loss_coef, n_layer=args.layers or 12, n_head=12, d_model=768, d_ffn=3072, seq_len=s,
                         moe_every=(args.moe_every if moe else 0), num_experts=args.experts_per_gpu * world, top_k=args.top_k,
                         capacity_factor=args.cf or None, ep_size=world, backend=backend, max_tokens=b * s, dtype=dtype)
        model = _GPTStep(GPTMoE(c, ep_group=ep_group, device=dev))
        ids = torch.randint(0, c.vocab_size, (b, s), generator=g)
        batch = {"ids": ids, "labels": ids.roll(-1, 1)}
    elif args.model == "bert":
        b, s = args.batch or 32, args.seq or 512
        c = BertMoEConfig(router_dtype=torch.float32 if args.router_fp32 else None, aux_loss_coef=args.aux_loss_coef,
                          z_loss_coef=args.z_loss_coef, n_layer=args.layers or 12, moe_layers=(2, 5, 8, 11) if moe else (), max_position=s,
                          num_experts=args.experts_per_gpu * world, top_k=args.top_k, capacity_factor=args.cf or None,
                          ep_size=world, backend=backend, max_tokens=b * s, dtype=dtype)
        model = _BertStep(BertMoEForQuestionAnswering(c, ep_group=ep_group, device=dev))
        batch = {"ids": torch.randint(0, c.vocab_size, (b, s), generator=g), "mask": torch.ones(b, s, dtype=torch.long),
                 "types": torch.zeros(b, s, dtype=torch.long), "start": torch.randint(0, s, (b,), generator=g),
                 "end": torch.randint(0, s, (b,), generator=g)}
    else:
        b, s = args.batch or 16, args.seq or 512
        c = TransformerXLMoEConfig(router_dtype=torch.float32 if args.router_fp32 else None, aux_loss_coef=args.aux_loss_coef,
                                   z_loss_coef=args.z_loss_coef, n_token=getattr(args, "n_token", 0) or 100, n_layer=args.layers or 12, tgt_len=s, mem_len=s, moe=moe,
                                   num_experts=args.experts_per_gpu * world, top_k=args.top_k,
                                   capacity_factor=args.cf or None, ep_size=world, backend=backend, max_tokens=b * s, dtype=dtype)
        model = _TXLStep(TransformerXLMoE(c, ep_group=ep_group, device=dev))
        batch = {"ids": torch.randint(1, 50, (b, s), generator=g), "labels": torch.randint(1, 50, (b, s), generator=g)}
    return model, {k: v.to(dev) for k, v in batch.items()}, b * s


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="gpt", choices=["gpt", "bert", "txl"])
    ap.add_argument("--variant", default="fused", choices=["dense", "nccl", "fused"])
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--experts-per-gpu", type=int, default=16)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--moe-every", type=int, default=1)
    ap.add_argument("--cf", type=float, default=0.0)
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--optimizer", default="sgd", choices=["sgd", "adamw"])
    ap.add_argument("--lr", type=float, default=1e-4)
    ap.add_argument("--aux-loss-coef", type=float, default=0.0, help="weight of the router load-balance loss")
    ap.add_argument("--z-loss-coef", type=float, default=0.0, help="weight of the router z-loss")
    ap.add_argument("--router-fp32", action="store_true", help="keep the routers in fp32")
    ap.add_argument("--fuse-expert-sgd", action="store_true",
                    help="fused variant with --optimizer sgd: expert weight matrices are updated inside the backward pass "
                         "(MoELayer.fuse_sgd; all of them when the experts live on one rank, the second projection otherwise)")
    ap.add_argument("--data", default="", help="txl only: training text file (word-level vocabulary built from it); "
                                               "default is a fixed synthetic batch")
    ap.add_argument("--valid", default="", help="txl only: validation text file, evaluated at the end")
    ap.add_argument("--ep-size", type=int, default=0,
                    help="ranks per expert-parallel group (default: all); the groups are data-parallel replicas of each other")
    ap.add_argument("--rebalance-every", type=int, default=0,
                    help="every N steps re-place the experts of each MoE layer from its last routing counts (0 = never)")
    ap.add_argument("--save", default="", help="checkpoint prefix written at the end (per-rank expert shards + manifest)")
    ap.add_argument("--save-every", type=int, default=0,
                    help="also write the checkpoint every N steps, so that a job restarted by the launcher "
                         "(torchrun --max-restarts) can pick up with --resume")
    ap.add_argument("--resume", default="", help="checkpoint prefix to load before training (any EP degree)")
    args = ap.parse_args()
    rank, _, world = init_distributed()
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    corpus = train_iter = None
    if args.data:
        if args.model != "txl":
            raise SystemExit("--data is supported for --model txl")
        from ..utils.data import Corpus
        corpus = Corpus(args.data, valid=args.valid or None)
        args.n_token = len(corpus.vocab)
    ep_size = args.ep_size or world
    ep_group = expert_dp_group = None
    if ep_size != world:
        from ..utils.dist import make_ep_dp_groups
        ep_group, expert_dp_group = make_ep_dp_groups(ep_size)
    model, batch, tokens = build(args, ep_size, dev, ep_group)
    wrapped = wrap_ddp(model) if world > 1 else model
    params = [p for p in model.parameters() if p.requires_grad]
    opt = torch.optim.SGD(params, lr=args.lr) if args.optimizer == "sgd" else torch.optim.AdamW(params, lr=args.lr)
    if args.fuse_expert_sgd:
        if args.variant != "fused" or args.optimizer != "sgd" or expert_dp_group is not None:
            raise SystemExit("--fuse-expert-sgd needs --variant fused, --optimizer sgd and experts that are not replicated")
        from ..layers import MoELayer
        for m in model.modules():
            if isinstance(m, MoELayer):
                m.fuse_sgd(args.lr)
    start_step = 0
    if args.resume:
        import os
        from ..utils.checkpoint import load_ep_checkpoint
        if os.path.exists(args.resume + ".manifest.json"):
            manifest = load_ep_checkpoint(model, args.resume, rank % ep_size, ep_size, optimizer=opt)
            start_step = int(manifest.get("extra", {}).get("step", 0))
            if rank == 0:
                print(f"resumed from {args.resume} at step {start_step}", flush=True)
        elif rank == 0:
            print(f"no checkpoint at {args.resume} yet: starting from scratch", flush=True)
    if corpus is not None:
        train_iter = corpus.iterator("train", args.batch or 16, args.seq or 512, device=dev, rank=rank, world=world)
        if len(train_iter) == 0:
            raise SystemExit("the training text is shorter than one batch of batch x seq tokens per rank")
    times = []
    import time
    for i in range(args.warmup + args.steps):
        if train_iter is not None:
            x, y = train_iter.get_batch(i % len(train_iter))
            if i % len(train_iter) == 0:
                model.mems = None                      # a new pass over the text: the recurrence memory starts over
            batch = {"ids": x, "labels": y}
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        if dev.type == "cuda":
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
        opt.zero_grad(set_to_none=True)
        loss = wrapped(batch)
        if (args.aux_loss_coef > 0 or args.z_loss_coef > 0) and args.variant != "dense":
            from ..layers import MoELayer
            for m in model.modules():
                if isinstance(m, MoELayer) and getattr(m.gate, "has_loss", False):
                    extra = m.gate.get_loss()
                    if extra is not None and extra.requires_grad:
                        loss = loss + extra.to(loss.dtype).sum()
        loss.backward()
        if expert_dp_group is not None and args.variant != "dense":
            from ..parallel.ddp import reduce_expert_grads
            reduce_expert_grads(model, expert_dp_group, scale=1.0 / world)   # replicas of an expert agree again
        opt.step()
        if args.rebalance_every > 0 and args.variant != "dense" and (i + 1) % args.rebalance_every == 0:
            from ..layers import MoELayer
            for m in model.modules():
                if isinstance(m, MoELayer) and m.count_table() is not None:
                    m.rebalance(optimizer=opt)     # collective; the cost lands in this step's time
        if dev.type == "cuda":
            e.record()
            torch.cuda.synchronize()
            ms = s.elapsed_time(e)
        else:
            ms = (time.perf_counter() - t0) * 1e3
        if i >= args.warmup:
            times.append(ms)
        if args.save and args.save_every > 0 and (i + 1) % args.save_every == 0 and rank < ep_size:
            from ..utils.checkpoint import save_ep_checkpoint
            save_ep_checkpoint(model, args.save, rank, ep_size, optimizer=opt,
                               extra={"model": args.model, "variant": args.variant, "step": start_step + i + 1})
        if rank == 0 and i % 10 == 0:
            print(f"STEP-{i}: step_time = {ms:.3f} ms, loss = {float(loss.detach()):.4f}", flush=True)
    avg = sum(times) / max(1, len(times))
    t = torch.tensor([avg], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(f"{args.variant} {args.model} {args.experts_per_gpu} [Summary] Average synchronized step_time = {float(t):.3f} ms")
        print(json.dumps({"bench": "e2e", "model": args.model, "variant": args.variant, "n_gpus": world,
                          "experts_per_gpu": args.experts_per_gpu, "step_ms": round(float(t), 3),
                          "tokens_per_s": round(tokens * world / float(t) * 1e3, 1), "final_loss": round(float(loss.detach()), 4)}))
    if corpus is not None and args.valid and corpus.data["valid"].numel() > (args.batch or 16) * ((args.seq or 512) + 1):
        from ..utils.data import evaluate_lm
        model.mems = None
        val = evaluate_lm(lambda x, y: model({"ids": x, "labels": y}),
                          corpus.iterator("valid", args.batch or 16, args.seq or 512, device=dev), max_batches=50)
        if rank == 0:
            print(json.dumps({"bench": "e2e", "model": args.model, "valid_loss": round(val, 4), "vocab": len(corpus.vocab)}))
    if args.save:
        from ..utils.checkpoint import save_ep_checkpoint
        if rank < ep_size:   # the other expert-parallel groups hold copies of the same shards
            save_ep_checkpoint(model, args.save, rank, ep_size, optimizer=opt,
                               extra={"model": args.model, "variant": args.variant, "step": start_step + args.warmup + args.steps})
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
