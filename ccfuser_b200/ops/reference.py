"""Dense single-process oracle of the whole expert-parallel layer.

The reference's numerics are not a usable oracle (fp16 accumulators at mix_moe/csrc/cuda/mix_gemm.cu:43,
dropped tail blocks at mix_gemm.cu:390-392, uninitialised bias gradients at mix_moe/csrc/mix_moe.h:342), so
every backend is tested against this plain fp32 loop over experts. It takes the inputs of *all* ranks and
the *full* expert weights and applies the same per-rank drop rule as the distributed code.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from ..gates import topk_softmax_reference
from .routing import route_local


def expert_ffn(x, w1, b1, w2, b2, activation: str, wg=None, bg=None):
    h = F.linear(x, w1, b1)
    if activation == "swiglu":
        h = F.silu(F.linear(x, wg, bg)) * h
    elif activation == "gelu":
        h = F.gelu(h)
    elif activation == "relu":
        h = F.relu(h)
    else:
        raise ValueError(activation)
    return F.linear(h, w2, b2)


def dense_moe_oracle(xs: List[torch.Tensor], params: Dict[str, torch.Tensor], *, top_k: int,
                     capacity: Optional[int], activation: str = "gelu", routing=None) -> List[torch.Tensor]:
    """xs: one [T_r, d] tensor per rank. params: full (all experts) tensors under the keys
    ``gate.weight [E,d]``, ``gate.bias [E]|None``, ``htoh4.weight [E,F,d]``, ``htoh4.bias``,
    ``h4toh.weight [E,d,F]``, ``h4toh.bias`` and for swiglu ``htoh4_gate.weight/bias``.
    Everything is computed in the dtype of ``params`` (use fp32/fp64). Differentiable.
    ``routing`` optionally gives one ``(idx [T,k], score [T,k])`` pair per rank instead of running the
    router (used to test expert kernels with the routing decisions of the implementation under test)."""
    gw, gb = params["gate.weight"], params.get("gate.bias")
    e_total = gw.shape[0]
    outs = []
    for x in xs:
        t, d = x.shape
        if routing is None:
            logits = F.linear(x.to(gw.dtype), gw, gb)
            idx, score = topk_softmax_reference(logits, top_k)
        else:
            idx, score = routing[len(outs)]
            idx = idx.to(torch.int64)
        score = score.to(gw.dtype)
        cap = capacity if capacity is not None else t * top_k
        plan = route_local(idx, e_total, cap)
        keep = plan.keep.view(t, top_k)
        y = torch.zeros(t, params["h4toh.weight"].shape[1], dtype=gw.dtype, device=x.device)
        for e in range(e_total):
            sel = (idx == e) & keep
            tok, slot = sel.nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            o = expert_ffn(
                x[tok].to(gw.dtype),
                params["htoh4.weight"][e], _opt(params, "htoh4.bias", e),
                params["h4toh.weight"][e], _opt(params, "h4toh.bias", e),
                activation,
                params["htoh4_gate.weight"][e] if activation == "swiglu" else None,
                _opt(params, "htoh4_gate.bias", e) if activation == "swiglu" else None)
            y = y.index_add(0, tok, o * score[tok, slot].unsqueeze(1))
        outs.append(y)
    return outs


def _opt(params, key, e):
    v = params.get(key)
    return None if v is None else v[e]


def _rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.detach().float(), b.detach().float()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-12))


def sampled_oracle_check(layer, x: torch.Tensor, idx: torch.Tensor, score: torch.Tensor, y: torch.Tensor,
                         gy: Optional[torch.Tensor] = None, dx: Optional[torch.Tensor] = None,
                         dscore: Optional[torch.Tensor] = None, n_sample: int = 64, expert: int = 0, group=None,
                         seed: int = 0) -> Dict[str, float]:
    """fp32 check of an MoE layer's result at a size where the dense oracle above would cost the full problem again:
    only ``n_sample`` tokens per rank are recomputed for the output (and for dx and the gate-weight gradient), and one
    local expert's rows for its weight gradients. Returns relative errors (max |a - b| / max |b|) under the keys
    ``y`` and, when ``gy`` is given, ``dx``, ``dscore``, ``dw1``, ``dw2`` (``dwg`` for SwiGLU, ``db*`` with biases).

    ``x [T, d]``, ``idx / score [T, k]`` are this rank's inputs and routing decisions, ``y [T, d]`` the layer's output
    for them; ``gy / dx / dscore`` the upstream gradient and the layer's gradients for x and score, with the expert
    parameters' ``.grad`` holding the rest. With a ``group`` of more than one rank the call is collective and covers the
    forward output only: every rank evaluates its own experts on all ranks' samples and the partial sums are
    all-reduced, so no weight leaves its owner.

    The drop rule is recomputed here from ``idx`` with ``route_local`` (not taken from the kernels under test)."""
    import torch.distributed as dist
    cfg = layer.config
    world = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
    rank = dist.get_rank(group) if world > 1 else 0
    e_loc, k, act = cfg.experts_per_rank, cfg.top_k, cfg.activation
    t, d = x.shape
    dev = x.device
    ex = layer.experts
    plan = route_local(idx, cfg.num_experts, cfg.capacity(t))
    keep = plan.keep.view(t, k)
    g = torch.Generator(device="cpu").manual_seed(seed + rank)
    samp = torch.randperm(t, generator=g)[:min(n_sample, t)].to(dev)
    ns = samp.numel()

    def expert_params(e_local: int, grad: bool):
        def f(m):
            w = m.weight[e_local].detach().float().requires_grad_(grad)
            b = None if m.bias is None else m.bias[e_local].detach().float().requires_grad_(grad)
            return w, b
        w1, b1 = f(ex.htoh4)
        w2, b2 = f(ex.h4toh)
        wg, bg = f(ex.htoh4_gate) if act == "swiglu" else (None, None)
        return w1, b1, w2, b2, wg, bg

    # ---- forward on the samples (all ranks' samples when distributed) -----------------------------------------
    xs = x[samp].detach().float()
    sidx = idx[samp].to(torch.int64)
    sw = torch.where(keep[samp], score[samp].detach().float(), torch.zeros((), device=dev))
    if world > 1:
        def gather(v):
            out = [torch.empty_like(v) for _ in range(world)]
            dist.all_gather(out, v.contiguous(), group=group)
            return torch.cat(out, 0)
        all_x, all_idx, all_w = gather(xs), gather(sidx), gather(sw)
    else:
        all_x, all_idx, all_w = xs, sidx, sw
    xs_g = all_x.clone().requires_grad_(gy is not None and world == 1)
    w_g = all_w.clone().requires_grad_(gy is not None and world == 1)
    part = torch.zeros(all_x.shape[0], d, dtype=torch.float32, device=dev)
    for el in range(e_loc):
        e = rank * e_loc + el
        tok, slot = ((all_idx == e) & (all_w != 0)).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        w1, b1, w2, b2, wg, bg = expert_params(el, False)
        o = expert_ffn(xs_g[tok], w1, b1, w2, b2, act, wg, bg)
        part = part.index_add(0, tok, o * w_g[tok, slot].unsqueeze(1))
    if world > 1:
        dist.all_reduce(part, group=group)
    mine = part[rank * ns:(rank + 1) * ns]
    out = {"y": _rel_err(y[samp], mine)}
    if gy is None or world > 1:
        return out
    # ---- backward on the samples: dx and the gradient of the gate weights ------------------------------------
    mine.backward(gy[samp].float())
    if dx is not None:
        out["dx"] = _rel_err(dx[samp], xs_g.grad)
    if dscore is not None:
        out["dscore"] = _rel_err(dscore[samp], w_g.grad)
    # ---- one expert's weight gradients from all of its rows -----------------------------------------------------
    tok, slot = ((idx.to(torch.int64) == expert) & keep).nonzero(as_tuple=True)
    w1, b1, w2, b2, wg, bg = expert_params(expert, True)
    o = expert_ffn(x[tok].detach().float(), w1, b1, w2, b2, act, wg, bg) * score[tok, slot].detach().float().unsqueeze(1)
    o.backward(gy[tok].float())
    out["dw1"] = _rel_err(ex.htoh4.weight.grad[expert], w1.grad)
    out["dw2"] = _rel_err(ex.h4toh.weight.grad[expert], w2.grad)
    if b1 is not None:
        out["db1"] = _rel_err(ex.htoh4.bias.grad[expert], b1.grad)
        out["db2"] = _rel_err(ex.h4toh.bias.grad[expert], b2.grad)
    if act == "swiglu":
        out["dwg"] = _rel_err(ex.htoh4_gate.weight.grad[expert], wg.grad)
        if bg is not None:
            out["dbg"] = _rel_err(ex.htoh4_gate.bias.grad[expert], bg.grad)
    return out
