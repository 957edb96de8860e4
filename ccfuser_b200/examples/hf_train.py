"""Hugging Face GPT-2 / BERT-QA with MoE FFN blocks, trained on synthetic batches: the literal counterpart of the
reference's end-to-end scripts (mix_moe/mix_moe/examples/models/moe_gpt_ddp.py: GPT-2 small, batch 8 x 1024, AdamW;
moe_bert_ddp.py: BertForQuestionAnswering, batch 32 x 512, MoE in layers 2, 5, 8, 11, 16 experts per GPU), using the
stock ``transformers`` classes converted in place (models/hf.py) instead of edited copies of the modelling files.
Weights are random-init from the configuration (no download).

    python -m ccfuser_b200.examples.hf_train --model gpt2 --variant fused --steps 20
    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 -m ccfuser_b200.examples.hf_train \
        --model bert --variant fused

Prints the reference's ``[Summary] Average synchronized step_time`` line and one JSON line.
"""
from __future__ import annotations

import argparse
import json
import time

import torch
import torch.distributed as dist

from ..models.hf import aux_loss, convert_bert, convert_gpt2
from ..parallel.ddp import wrap_ddp
from ..utils.dist import init_distributed


def build(args, world, dev, dtype):
    from transformers import BertConfig, BertForQuestionAnswering, GPT2Config, GPT2LMHeadModel
    backend = {"dense": None, "nccl": "nccl", "fused": "fused"}[args.variant]
    if dev.type != "cuda" and backend is not None:
        backend = "cpu"
    g = torch.Generator().manual_seed(1 + (dist.get_rank() if dist.is_initialized() else 0))
    if args.model == "gpt2":
        b, s = args.batch or 8, args.seq or 1024
        cfg = GPT2Config(n_layer=args.layers or 12, n_head=args.heads or 12, n_embd=args.hidden or 768, n_positions=s,
                         vocab_size=args.vocab or 50257, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
        model = GPT2LMHeadModel(cfg).to(device=dev, dtype=dtype)
        layers = [] if backend is None else convert_gpt2(
            model, num_experts=args.experts_per_gpu * world, top_k=args.top_k, every=args.moe_every, backend=backend,
            max_tokens=b * s, capacity_factor=args.cf or None)
        ids = torch.randint(0, cfg.vocab_size, (b, s), generator=g).to(dev)
        batch = dict(input_ids=ids, labels=ids)
    else:
        b, s = args.batch or 32, args.seq or 512
        cfg = BertConfig(num_hidden_layers=args.layers or 12, num_attention_heads=args.heads or 12,
                         hidden_size=args.hidden or 768, intermediate_size=4 * (args.hidden or 768),
                         vocab_size=args.vocab or 30522, max_position_embeddings=s, hidden_dropout_prob=0.0,
                         attention_probs_dropout_prob=0.0)
        model = BertForQuestionAnswering(cfg).to(device=dev, dtype=dtype)
        layers = [] if backend is None else convert_bert(
            model, num_experts=args.experts_per_gpu * world, top_k=args.top_k, layers=(2, 5, 8, 11), backend=backend,
            max_tokens=b * s, capacity_factor=args.cf or None)
        batch = dict(input_ids=torch.randint(0, cfg.vocab_size, (b, s), generator=g).to(dev),
                     attention_mask=torch.ones(b, s, dtype=torch.long, device=dev),
                     start_positions=torch.randint(0, s, (b,), generator=g).to(dev),
                     end_positions=torch.randint(0, s, (b,), generator=g).to(dev))
    return model, layers, batch, b * s


class _LossOnly(torch.nn.Module):
    """DistributedDataParallel wants tensors out of forward; Hugging Face models return a ModelOutput."""

    def __init__(self, model):
        super().__init__()
        self.model = model

    def forward(self, **batch):
        return self.model(**batch).loss


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="gpt2", choices=["gpt2", "bert"])
    ap.add_argument("--variant", default="fused", choices=["dense", "nccl", "fused"])
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--heads", type=int, default=0)
    ap.add_argument("--hidden", type=int, default=0)
    ap.add_argument("--vocab", type=int, default=0)
    ap.add_argument("--experts-per-gpu", type=int, default=16)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--moe-every", type=int, default=1)
    ap.add_argument("--cf", type=float, default=0.0)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"])
    ap.add_argument("--lr", type=float, default=1e-4)
    args = ap.parse_args(argv)
    rank, _, world = init_distributed()
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dtype]
    model, layers, batch, tokens = build(args, world, dev, dtype)
    wrapped = wrap_ddp(_LossOnly(model)) if world > 1 else _LossOnly(model)
    opt = torch.optim.AdamW([p for p in model.parameters() if p.requires_grad], lr=args.lr)
    times = []
    loss = None
    for i in range(args.warmup + args.steps):
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        if dev.type == "cuda":
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
        opt.zero_grad(set_to_none=True)
        loss = wrapped(**batch)
        extra = aux_loss(layers)
        if extra is not None and extra.requires_grad:
            loss = loss + extra.to(loss.dtype).sum()
        loss.backward()
        opt.step()
        if dev.type == "cuda":
            e.record()
            torch.cuda.synchronize()
            ms = s.elapsed_time(e)
        else:
            ms = (time.perf_counter() - t0) * 1e3
        if i >= args.warmup:
            times.append(ms)
    for layer in layers:
        layer.check_status()
    avg = sum(times) / max(1, len(times))
    t = torch.tensor([avg], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    out = {"bench": "e2e_hf", "model": args.model, "variant": args.variant, "n_gpus": world,
           "experts_per_gpu": args.experts_per_gpu, "moe_layers": len(layers), "step_ms": round(float(t), 3),
           "tokens_per_s": round(tokens * world / float(t) * 1e3, 1), "final_loss": round(float(loss.detach()), 4)}
    if rank == 0:
        print(f"{args.variant} {args.model} {args.experts_per_gpu} [Summary] Average synchronized step_time = {float(t):.3f} ms")
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return out


if __name__ == "__main__":
    main()
