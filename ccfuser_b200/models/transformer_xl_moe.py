"""Transformer-XL language model (segment recurrence + relative positional attention) with an MoE FFN in every
decoder layer.

The reference patches the original Transformer-XL code: ``CustomizedMoEPositionwiseFF`` subclasses its MoE layer
and replaces ``PositionwiseFF`` in every ``RelPartialLearnableDecoderLayer``
(mix_moe/mix_moe/examples/transformer-xl/mem_transformer_mix_moe.py:383-419,478-485); training uses synthetic ids
over a 100-token vocabulary, 12 layers, d_model 512, 8 heads, d_inner 2048, tgt_len = mem_len = 512
(mix_moe/ae/fig11_data.sh:52-92, mix_moe/mix_moe/examples/transformer-xl/train_ddp.py:228,360-361).
This module is a compact re-implementation of that architecture: batch-first tensors, the standard
``rel_shift`` formulation of (q + u) k^T + (q + v) r^T, cached hidden states as memory, plain or adaptive softmax.
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import MoEConfig
from ..layers import MoELayer
from ..ops.norm import LayerNorm


@dataclasses.dataclass
class TransformerXLMoEConfig:
    """Transformer-XL with relative positions and segment memory; ``moe=True`` puts an MoE layer in every decoder layer
    (the reference's end-to-end configuration: 12 layers, d_model 512, 8 heads, d_inner 2048, tgt_len = mem_len = 512)."""
    n_token: int = 100
    n_layer: int = 12
    n_head: int = 8
    d_model: int = 512
    d_head: int = 64
    d_inner: int = 2048
    tgt_len: int = 512
    mem_len: int = 512
    moe: bool = True
    num_experts: int = 16
    top_k: int = 2
    capacity_factor: Optional[float] = None
    ep_size: int = 1
    backend: str = "auto"
    max_tokens: int = 16 * 512
    dtype: torch.dtype = torch.bfloat16
    pre_lnorm: bool = False
    adaptive_cutoffs: Sequence[int] = ()
    dropout: float = 0.0

    router_dtype: Optional[torch.dtype] = None
    aux_loss_coef: float = 0.0
    z_loss_coef: float = 0.0

    def moe_config(self) -> MoEConfig:
        return MoEConfig(d_model=self.d_model, d_ffn=self.d_inner, num_experts=self.num_experts, top_k=self.top_k,
                         capacity_factor=self.capacity_factor, activation="relu", dtype=self.dtype,
                         ep_size=self.ep_size, backend=self.backend, max_tokens=self.max_tokens,
                         router_dtype=self.router_dtype, aux_loss_coef=self.aux_loss_coef, z_loss_coef=self.z_loss_coef)


class PositionalEmbedding(nn.Module):
    """Sinusoidal embedding of relative positions."""
    def __init__(self, d, device=None):
        super().__init__()
        self.register_buffer("inv_freq", 1.0 / (10000 ** (torch.arange(0.0, d, 2.0, device=device) / d)),
                             persistent=False)

    def forward(self, pos_seq):
        s = torch.outer(pos_seq, self.inv_freq.to(pos_seq.device))
        return torch.cat([s.sin(), s.cos()], dim=-1)


class PositionwiseFF(nn.Module):
    """The dense feed-forward block (used when ``moe=False``)."""
    def __init__(self, c: TransformerXLMoEConfig, device=None):
        super().__init__()
        self.fc = nn.Linear(c.d_model, c.d_inner, device=device, dtype=c.dtype)
        self.proj = nn.Linear(c.d_inner, c.d_model, device=device, dtype=c.dtype)

    def forward(self, x):
        return self.proj(F.relu(self.fc(x)))


def _rel_shift(x):
    """x [B, H, Q, K] scores indexed by relative distance -> aligned with absolute key positions."""
    b, h, q, k = x.shape
    x = F.pad(x, (1, 0))
    x = x.view(b, h, k + 1, q)[:, :, 1:].reshape(b, h, q, k)
    return x


class RelPartialLearnableAttention(nn.Module):
    """Multi-head attention over [memory, segment] with Transformer-XL's relative position terms (content and position
    biases u, v; relative shift)."""
    def __init__(self, c: TransformerXLMoEConfig, device=None):
        super().__init__()
        self.n_head, self.d_head = c.n_head, c.d_head
        hd = c.n_head * c.d_head
        self.qkv_net = nn.Linear(c.d_model, 3 * hd, bias=False, device=device, dtype=c.dtype)
        self.r_net = nn.Linear(c.d_model, hd, bias=False, device=device, dtype=c.dtype)
        self.o_net = nn.Linear(hd, c.d_model, bias=False, device=device, dtype=c.dtype)
        self.scale = 1.0 / (c.d_head ** 0.5)

    def forward(self, x, r, r_w_bias, r_r_bias, mask, mem):
        b, q, _ = x.shape
        cat = x if mem is None or mem.shape[1] == 0 else torch.cat([mem.to(x.dtype), x], 1)
        k_len = cat.shape[1]
        heads = self.qkv_net(cat).view(b, k_len, 3, self.n_head, self.d_head)
        wq = heads[:, -q:, 0]                                   # [B, Q, H, Dh]
        wk, wv = heads[:, :, 1], heads[:, :, 2]                 # [B, K, H, Dh]
        rk = self.r_net(r).view(k_len, self.n_head, self.d_head)  # [K, H, Dh]
        ac = torch.einsum("bqhd,bkhd->bhqk", wq + r_w_bias, wk)
        bd = _rel_shift(torch.einsum("bqhd,khd->bhqk", wq + r_r_bias, rk))
        score = (ac + bd) * self.scale
        score = score.float().masked_fill(mask, float("-inf"))
        prob = torch.softmax(score, dim=-1).to(x.dtype)
        out = torch.einsum("bhqk,bkhd->bqhd", prob, wv).reshape(b, q, self.n_head * self.d_head)
        return self.o_net(out)


class DecoderLayer(nn.Module):
    """Attention with memory, then the position-wise FFN (dense or MoE)."""
    def __init__(self, c: TransformerXLMoEConfig, ep_group=None, device=None):
        super().__init__()
        self.attn = RelPartialLearnableAttention(c, device)
        self.ln1 = LayerNorm(c.d_model, device=device, dtype=c.dtype)
        self.ln2 = LayerNorm(c.d_model, device=device, dtype=c.dtype)
        self.is_moe = c.moe
        self.pos_ff = MoELayer(c.moe_config(), ep_group=ep_group, device=device) if c.moe else PositionwiseFF(c, device)
        self.pre_lnorm = c.pre_lnorm

    def forward(self, x, r, r_w_bias, r_r_bias, mask, mem):
        if self.pre_lnorm:
            x = x + self.attn(self.ln1(x), r, r_w_bias, r_r_bias, mask, None if mem is None else self.ln1(mem))
            return x + self.pos_ff(self.ln2(x))
        x = self.ln1(x + self.attn(x, r, r_w_bias, r_r_bias, mask, mem))
        return self.ln2(x + self.pos_ff(x))


class TransformerXLMoE(nn.Module):
    """``forward(data [B, T], target [B, T], mems=None)`` -> (mean loss, new_mems)."""

    def __init__(self, c: TransformerXLMoEConfig, ep_group=None, device=None):
        super().__init__()
        self.config = c
        self.word_emb = nn.Embedding(c.n_token, c.d_model, device=device, dtype=c.dtype)
        self.pos_emb = PositionalEmbedding(c.d_model, device)
        self.r_w_bias = nn.Parameter(torch.zeros(c.n_head, c.d_head, device=device, dtype=c.dtype))
        self.r_r_bias = nn.Parameter(torch.zeros(c.n_head, c.d_head, device=device, dtype=c.dtype))
        self.layers = nn.ModuleList([DecoderLayer(c, ep_group, device) for _ in range(c.n_layer)])
        self.emb_scale = c.d_model ** 0.5
        if c.adaptive_cutoffs:
            self.crit = nn.AdaptiveLogSoftmaxWithLoss(c.d_model, c.n_token, list(c.adaptive_cutoffs), device=device)
        else:
            self.crit = None
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, std=0.02)
            if type(m).__name__ == "ExpertLinear":
                nn.init.normal_(m.weight, std=0.02)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)
        nn.init.normal_(self.r_w_bias, std=0.02)
        nn.init.normal_(self.r_r_bias, std=0.02)

    def init_mems(self, batch, device):
        c = self.config
        if c.mem_len <= 0:
            return None
        return [torch.zeros(batch, 0, c.d_model, dtype=c.dtype, device=device) for _ in range(c.n_layer)]

    def _update_mems(self, hids: List[torch.Tensor], mems, q_len):
        if mems is None:
            return None
        with torch.no_grad():
            new = []
            for h, m in zip(hids, mems):
                cat = torch.cat([m, h], 1)
                new.append(cat[:, -self.config.mem_len:].detach())
        return new

    def forward(self, data, target=None, mems=None):
        b, q = data.shape
        if mems is None:
            mems = self.init_mems(b, data.device)
        m_len = mems[0].shape[1] if mems is not None else 0
        k_len = m_len + q
        x = self.word_emb(data) * self.emb_scale
        pos_seq = torch.arange(k_len - 1, -1, -1.0, device=data.device)
        r = self.pos_emb(pos_seq).to(x.dtype)
        mask = torch.triu(torch.ones(q, k_len, device=data.device, dtype=torch.bool), diagonal=1 + m_len)[None, None]
        hids = []
        for i, layer in enumerate(self.layers):
            hids.append(x)
            x = layer(x, r, self.r_w_bias, self.r_r_bias, mask, None if mems is None else mems[i])
        new_mems = self._update_mems(hids, mems, q)
        if target is None:
            return x, new_mems
        if self.crit is not None:
            loss = self.crit(x.reshape(-1, x.shape[-1]).float(), target.reshape(-1)).loss
        else:
            logits = F.linear(x, self.word_emb.weight).float()
            loss = F.cross_entropy(logits.view(-1, logits.shape[-1]), target.reshape(-1))
        return loss, new_mems

    def moe_layers(self):
        return [l.pos_ff for l in self.layers if l.is_moe]
