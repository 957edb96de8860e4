"""GPT-style decoder with MoE FFNs (the end-to-end training workload).

The reference patches a Hugging Face GPT-2 by swapping ``transformer.h.<i>.mlp`` for its MoE layer
(mix_moe/mix_moe/examples/models/moe_gpt_ddp.py:207-215, with the wrong module path at :318 so that its
published GPT numbers contain no MoE layer). This is a self-contained pre-LN GPT-2 architecture with the
same knobs: learned positions, tied embedding / LM head, causal attention, GELU FFN, and an
``MoELayer`` in place of the FFN of every ``moe_every``-th block.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import MoEConfig
from ..layers import MoELayer
from ..ops.norm import LayerNorm


@dataclasses.dataclass
class GPTMoEConfig:
    """GPT-2 style decoder with an MoE FFN in every ``moe_every``-th block; the defaults are the benchmark model
    (24 layers, d_model 2048, 16 heads, seq 1024, 64 experts, top-2, FFN 8192, GELU)."""
    vocab_size: int = 50257
    n_layer: int = 24
    n_head: int = 16
    d_model: int = 2048
    d_ffn: int = 8192
    seq_len: int = 1024
    moe_every: int = 2            # block i has an MoE FFN when i % moe_every == moe_every - 1; 0 = dense model
    num_experts: int = 64
    top_k: int = 2
    capacity_factor: Optional[float] = None
    activation: str = "gelu"
    ep_size: int = 1
    backend: str = "auto"
    max_tokens: int = 8192        # tokens per rank per step (batch * seq_len)
    dtype: torch.dtype = torch.bfloat16
    recv_factor: float = 2.0      # receive-buffer size of a rank relative to the balanced load (no capacity factor)

    router_dtype: Optional[torch.dtype] = None
    aux_loss_coef: float = 0.0
    z_loss_coef: float = 0.0

    def moe_config(self) -> MoEConfig:
        return MoEConfig(d_model=self.d_model, d_ffn=self.d_ffn, num_experts=self.num_experts, top_k=self.top_k,
                         capacity_factor=self.capacity_factor, activation=self.activation, dtype=self.dtype,
                         ep_size=self.ep_size, backend=self.backend, max_tokens=self.max_tokens, recv_factor=self.recv_factor,
                         router_dtype=self.router_dtype, aux_loss_coef=self.aux_loss_coef, z_loss_coef=self.z_loss_coef)

    def flops_per_token(self) -> float:
        """Forward+backward model FLOPs per token (3 x forward; attention scores included)."""
        d, f, s = self.d_model, self.d_ffn, self.seq_len
        attn = 2 * 4 * d * d + 2 * 2 * s * d
        ffn_mult = 3 if self.activation == "swiglu" else 2
        dense_ffn = 2 * ffn_mult * d * f
        n_moe = sum(1 for i in range(self.n_layer) if self.is_moe(i))
        fwd = self.n_layer * attn + (self.n_layer - n_moe) * dense_ffn + n_moe * self.top_k * dense_ffn
        fwd += n_moe * 2 * d * self.num_experts + 2 * d * self.vocab_size
        return 3.0 * fwd

    def is_moe(self, i: int) -> bool:
        return self.moe_every > 0 and i % self.moe_every == self.moe_every - 1


class CausalSelfAttention(nn.Module):
    """Causal multi-head attention. Query, key and value have their own projections: with one fused QKV matrix the
    backward pass has to concatenate the three gradients again (a 100 MB copy per layer at the benchmark size)."""

    def __init__(self, c: GPTMoEConfig, device=None):
        super().__init__()
        self.n_head = c.n_head
        self.q_proj = nn.Linear(c.d_model, c.d_model, device=device, dtype=c.dtype)
        self.k_proj = nn.Linear(c.d_model, c.d_model, device=device, dtype=c.dtype)
        self.v_proj = nn.Linear(c.d_model, c.d_model, device=device, dtype=c.dtype)
        self.c_proj = nn.Linear(c.d_model, c.d_model, device=device, dtype=c.dtype)

    def forward(self, x):
        b, s, d = x.shape
        h = self.n_head
        q = self.q_proj(x).view(b, s, h, d // h).transpose(1, 2)
        k = self.k_proj(x).view(b, s, h, d // h).transpose(1, 2)
        v = self.v_proj(x).view(b, s, h, d // h).transpose(1, 2)
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.c_proj(y.transpose(1, 2).reshape(b, s, d))


class DenseFFN(nn.Module):
    """The ordinary (non-MoE) feed-forward block of the same shape as one expert."""
    def __init__(self, c: GPTMoEConfig, device=None):
        super().__init__()
        self.act = c.activation
        self.c_fc = nn.Linear(c.d_model, c.d_ffn, device=device, dtype=c.dtype)
        if self.act == "swiglu":
            self.c_gate = nn.Linear(c.d_model, c.d_ffn, device=device, dtype=c.dtype)
        self.c_proj = nn.Linear(c.d_ffn, c.d_model, device=device, dtype=c.dtype)

    def forward(self, x):
        h = self.c_fc(x)
        if self.act == "swiglu":
            h = F.silu(self.c_gate(x)) * h
        elif self.act == "relu":
            h = F.relu(h)
        else:
            h = F.gelu(h)
        return self.c_proj(h)


class Block(nn.Module):
    """Pre-LN transformer block: attention, then a dense FFN or an MoE layer."""
    def __init__(self, c: GPTMoEConfig, moe: bool, ep_group=None, device=None):
        super().__init__()
        self.ln_1 = LayerNorm(c.d_model, device=device, dtype=c.dtype)
        self.attn = CausalSelfAttention(c, device)
        self.ln_2 = LayerNorm(c.d_model, device=device, dtype=c.dtype)
        self.is_moe = moe
        self.mlp = MoELayer(c.moe_config(), ep_group=ep_group, device=device) if moe else DenseFFN(c, device)

    def forward(self, x):
        x = x + self.attn(self.ln_1(x))
        return x + self.mlp(self.ln_2(x))


class GPTMoE(nn.Module):
    """``forward(ids [B,S], labels=None)`` -> logits, or the mean next-token cross-entropy when labels are given."""

    def __init__(self, c: GPTMoEConfig, ep_group=None, device=None):
        super().__init__()
        self.config = c
        # the embedding / LM-head matrix is padded to a multiple of 128 rows so the vocabulary GEMM runs on an
        # aligned tensor-core kernel; the padding columns of the logits are masked out of the softmax
        self.vocab_padded = (c.vocab_size + 127) // 128 * 128
        self.wte = nn.Embedding(self.vocab_padded, c.d_model, device=device, dtype=c.dtype)
        self.wpe = nn.Embedding(c.seq_len, c.d_model, device=device, dtype=c.dtype)
        self.h = nn.ModuleList([Block(c, c.is_moe(i), ep_group, device) for i in range(c.n_layer)])
        self.ln_f = LayerNorm(c.d_model, device=device, dtype=c.dtype)
        self.apply(self._init)
        for name, p in self.named_parameters():
            if name.endswith("c_proj.weight"):
                nn.init.normal_(p, mean=0.0, std=0.02 / math.sqrt(2 * c.n_layer))

    @staticmethod
    def _init(m):
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, mean=0.0, std=0.02)
            if m.bias is not None:
                nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, mean=0.0, std=0.02)
        elif type(m).__name__ == "ExpertLinear":
            nn.init.normal_(m.weight, mean=0.0, std=0.02)
            if m.bias is not None:
                nn.init.zeros_(m.bias)

    def forward(self, ids: torch.Tensor, labels: Optional[torch.Tensor] = None):
        b, s = ids.shape
        pos = torch.arange(s, device=ids.device)
        x = self.wte(ids) + self.wpe(pos)
        for blk in self.h:
            x = blk(x)
        x = self.ln_f(x)
        logits = F.linear(x, self.wte.weight)
        if self.vocab_padded != self.config.vocab_size:
            logits[..., self.config.vocab_size:] = float("-inf")
        if labels is None:
            return logits[..., :self.config.vocab_size]
        return F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), labels.reshape(-1))

    def moe_layers(self):
        return [blk.mlp for blk in self.h if blk.is_moe]

    def aux_loss(self):
        losses = [m.gate.get_loss() for m in self.moe_layers() if getattr(m.gate, "has_loss", False)]
        losses = [l for l in losses if l is not None]
        return sum(losses) if losses else None
