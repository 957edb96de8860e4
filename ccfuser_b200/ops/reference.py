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
