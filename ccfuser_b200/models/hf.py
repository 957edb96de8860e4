"""Turn the feed-forward blocks of Hugging Face GPT-2 and BERT models into expert-parallel MoE layers.

The reference's end-to-end experiments run on edited copies of Hugging Face's modelling files in which selected
``mlp`` / ``ffn`` blocks are replaced by its MoE layer (GPT-2: mix_moe/mix_moe/examples/models/moe_gpt.py:583-592 and
:1200-1203 for the DDP ignore list; BERT-QA: mix_moe/mix_moe/examples/models/moe_bert.py:557-566, layers 2, 5, 8, 11 at
mix_moe/mix_moe/examples/models/moe_bert_ddp.py:406-417). Here the stock ``transformers`` classes are converted in place,
so no modelling file has to be vendored:

    model = GPT2LMHeadModel(config)
    layers = convert_gpt2(model, num_experts=64, top_k=2, every=2, ep_group=group, device="cuda")
    model = wrap_ddp(model)              # expert parameters are already tagged for the ignore list

``transformers`` is imported only by the caller; this module looks at attribute names, not classes.
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence

import torch
import torch.nn as nn

from ..config import MoEConfig
from ..layers import MoELayer


class MoEMLP(nn.Module):
    """Drop-in for a transformer block's MLP: ``hidden -> hidden`` through an MoE layer, then the block's dropout."""

    def __init__(self, moe: MoELayer, dropout: float = 0.0):
        super().__init__()
        self.moe = moe
        self.dropout = nn.Dropout(dropout)

    def forward(self, hidden_states, *args, **kwargs):
        return self.dropout(self.moe(hidden_states))


class _PassThrough(nn.Module):
    """Stands in for the dense projection of BertOutput once the MoE layer already returns hidden-size rows."""

    def forward(self, x):
        return x


def _make_layer(d_model: int, d_ffn: int, num_experts: int, top_k: int, activation: str, capacity_factor, ep_group,
                ep_size: int, backend: str, max_tokens: int, dtype, device) -> MoELayer:
    cfg = MoEConfig(d_model=d_model, d_ffn=d_ffn, num_experts=num_experts, top_k=top_k, capacity_factor=capacity_factor,
                    activation=activation, dtype=dtype, ep_size=ep_size, backend=backend, max_tokens=max_tokens)
    return MoELayer(cfg, ep_group=ep_group, device=device)


def _ep_size(ep_group) -> int:
    import torch.distributed as dist
    return dist.get_world_size(ep_group) if dist.is_initialized() else 1


def _pick(n_layers: int, every: int, layers: Optional[Iterable[int]]) -> List[int]:
    if layers is not None:
        sel = sorted(set(int(i) for i in layers))
        if sel and (sel[0] < 0 or sel[-1] >= n_layers):
            raise ValueError(f"layer indices must be in [0, {n_layers})")
        return sel
    # "an MoE FFN every `every` layers", counted so that the last layer of each group is the MoE one
    return [i for i in range(n_layers) if (i + 1) % every == 0]


def convert_gpt2(model: nn.Module, *, num_experts: int, top_k: int = 2, every: int = 2,
                 layers: Optional[Sequence[int]] = None, d_ffn: Optional[int] = None, activation: str = "gelu",
                 capacity_factor: Optional[float] = None, ep_group=None, backend: str = "auto",
                 max_tokens: int = 8192, dtype=None, device=None) -> List[MoELayer]:
    """Replace ``block.mlp`` of the chosen GPT-2 blocks (``model.transformer.h`` or ``model.h``) by MoE layers.
    Returns the new layers in block order."""
    body = getattr(model, "transformer", model)
    blocks = getattr(body, "h", None)
    if blocks is None:
        raise TypeError("expected a GPT-2 style model with .transformer.h (or .h) blocks")
    cfg = model.config
    d_model = cfg.n_embd
    inner = d_ffn or getattr(cfg, "n_inner", None) or 4 * d_model
    p0 = next(model.parameters())
    dtype = dtype or p0.dtype
    device = device if device is not None else p0.device
    out = []
    for i in _pick(len(blocks), every, layers):
        moe = _make_layer(d_model, inner, num_experts, top_k, activation, capacity_factor, ep_group, _ep_size(ep_group),
                          backend, max_tokens, dtype, device)
        blocks[i].mlp = MoEMLP(moe, getattr(cfg, "resid_pdrop", 0.0))
        out.append(moe)
    return out


def convert_bert(model: nn.Module, *, num_experts: int, top_k: int = 2, layers: Sequence[int] = (2, 5, 8, 11),
                 d_ffn: Optional[int] = None, activation: str = "gelu", capacity_factor: Optional[float] = None,
                 ep_group=None, backend: str = "auto", max_tokens: int = 16384, dtype=None, device=None) -> List[MoELayer]:
    """Replace the feed-forward part of the chosen BERT encoder layers. In Hugging Face's BertLayer the FFN is split
    into ``intermediate`` (dense + activation) and ``output`` (dense + dropout + residual LayerNorm): the MoE layer
    takes the place of ``intermediate`` and of ``output.dense``; dropout, residual and LayerNorm stay."""
    body = getattr(model, "bert", model)
    enc = getattr(getattr(body, "encoder", None), "layer", None)
    if enc is None:
        raise TypeError("expected a BERT style model with .bert.encoder.layer (or .encoder.layer)")
    cfg = model.config
    d_model = cfg.hidden_size
    inner = d_ffn or cfg.intermediate_size
    p0 = next(model.parameters())
    dtype = dtype or p0.dtype
    device = device if device is not None else p0.device
    out = []
    for i in _pick(len(enc), 1, [l for l in layers if l < len(enc)]):
        moe = _make_layer(d_model, inner, num_experts, top_k, activation, capacity_factor, ep_group, _ep_size(ep_group),
                          backend, max_tokens, dtype, device)
        enc[i].intermediate = MoEMLP(moe, 0.0)
        enc[i].output.dense = _PassThrough()
        out.append(moe)
    return out


def aux_loss(layers: Iterable[MoELayer]):
    """Sum of the load-balance losses the gates of ``layers`` recorded in their last forward (None if there is none)."""
    total = None
    for layer in layers:
        gate = layer.gate
        loss = gate.get_loss(clear=True) if hasattr(gate, "get_loss") else None
        if loss is not None:
            total = loss if total is None else total + loss
    return total
