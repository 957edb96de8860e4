"""BERT encoder with MoE FFNs and a question-answering head.

The reference wraps Hugging Face's BertForQuestionAnswering and swaps ``bert.encoder.layer.<i>.ffn`` of layers
2, 5, 8 and 11 for its MoE layer (mix_moe/mix_moe/examples/models/moe_bert_ddp.py:314,406-417, FFN wrapper at
mix_moe/mix_moe/examples/models/moe_bert.py:557-566). This is a self-contained post-LN BERT with the same
structure: word/position/type embeddings, bidirectional attention with a padding mask, GELU FFN, and a
span head producing start/end logits.
"""
from __future__ import annotations

import dataclasses
from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import MoEConfig
from ..layers import MoELayer
from ..ops.norm import LayerNorm


@dataclasses.dataclass
class BertMoEConfig:
    """BERT-base sized encoder; ``moe_layers`` lists the layers whose FFN is an MoE layer (the reference uses 2, 5, 8, 11)."""
    vocab_size: int = 30522
    n_layer: int = 12
    n_head: int = 12
    d_model: int = 768
    d_ffn: int = 3072
    max_position: int = 512
    type_vocab_size: int = 2
    moe_layers: Sequence[int] = (2, 5, 8, 11)
    num_experts: int = 16
    top_k: int = 2
    capacity_factor: Optional[float] = None
    ep_size: int = 1
    backend: str = "auto"
    max_tokens: int = 32 * 512
    dtype: torch.dtype = torch.bfloat16
    layer_norm_eps: float = 1e-12

    router_dtype: Optional[torch.dtype] = None
    aux_loss_coef: float = 0.0
    z_loss_coef: float = 0.0

    def moe_config(self) -> MoEConfig:
        return MoEConfig(d_model=self.d_model, d_ffn=self.d_ffn, num_experts=self.num_experts, top_k=self.top_k,
                         capacity_factor=self.capacity_factor, activation="gelu", dtype=self.dtype,
                         ep_size=self.ep_size, backend=self.backend, max_tokens=self.max_tokens,
                         router_dtype=self.router_dtype, aux_loss_coef=self.aux_loss_coef, z_loss_coef=self.z_loss_coef)


class BertSelfAttention(nn.Module):
    """Bidirectional multi-head attention with a key padding mask."""
    def __init__(self, c: BertMoEConfig, device=None):
        super().__init__()
        self.n_head = c.n_head
        self.qkv = nn.Linear(c.d_model, 3 * c.d_model, device=device, dtype=c.dtype)
        self.out = nn.Linear(c.d_model, c.d_model, device=device, dtype=c.dtype)

    def forward(self, x, mask):
        b, s, d = x.shape
        q, k, v = self.qkv(x).view(b, s, 3, self.n_head, d // self.n_head).permute(2, 0, 3, 1, 4)
        y = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
        return self.out(y.transpose(1, 2).reshape(b, s, d))


class FFN(nn.Module):
    """Dense intermediate + output projection (the module the reference replaces, moe_bert.py:557-566)."""

    def __init__(self, c: BertMoEConfig, device=None):
        super().__init__()
        self.fc = nn.Linear(c.d_model, c.d_ffn, device=device, dtype=c.dtype)
        self.proj = nn.Linear(c.d_ffn, c.d_model, device=device, dtype=c.dtype)

    def forward(self, x):
        return self.proj(F.gelu(self.fc(x)))


class BertLayer(nn.Module):
    """Post-LN encoder layer: attention + residual LayerNorm, FFN (dense or MoE) + residual LayerNorm."""
    def __init__(self, c: BertMoEConfig, moe: bool, ep_group=None, device=None):
        super().__init__()
        self.attention = BertSelfAttention(c, device)
        self.ln_attn = LayerNorm(c.d_model, eps=c.layer_norm_eps, device=device, dtype=c.dtype)
        self.is_moe = moe
        self.ffn = MoELayer(c.moe_config(), ep_group=ep_group, device=device) if moe else FFN(c, device)
        self.ln_ffn = LayerNorm(c.d_model, eps=c.layer_norm_eps, device=device, dtype=c.dtype)

    def forward(self, x, mask, token_mask=None):
        x = self.ln_attn(x + self.attention(x, mask))
        # padding tokens skip the experts (their FFN output is zero; nothing downstream reads those positions)
        ffn = self.ffn(x, token_mask=token_mask) if (self.is_moe and token_mask is not None) else self.ffn(x)
        return self.ln_ffn(x + ffn)


class BertMoEForQuestionAnswering(nn.Module):
    """``forward(input_ids, attention_mask=None, token_type_ids=None, start_positions=None, end_positions=None)``
    returns ``(start_logits, end_logits)`` or the span loss when both positions are given."""

    def __init__(self, c: BertMoEConfig, ep_group=None, device=None):
        super().__init__()
        self.config = c
        self.word = nn.Embedding(c.vocab_size, c.d_model, device=device, dtype=c.dtype)
        self.position = nn.Embedding(c.max_position, c.d_model, device=device, dtype=c.dtype)
        self.token_type = nn.Embedding(c.type_vocab_size, c.d_model, device=device, dtype=c.dtype)
        self.ln_emb = LayerNorm(c.d_model, eps=c.layer_norm_eps, device=device, dtype=c.dtype)
        self.layer = nn.ModuleList([BertLayer(c, i in set(c.moe_layers), ep_group, device) for i in range(c.n_layer)])
        self.qa_outputs = nn.Linear(c.d_model, 2, device=device, dtype=c.dtype)
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, std=0.02)
            if type(m).__name__ == "ExpertLinear":
                nn.init.normal_(m.weight, std=0.02)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, start_positions=None, end_positions=None):
        b, s = input_ids.shape
        pos = torch.arange(s, device=input_ids.device)
        tt = token_type_ids if token_type_ids is not None else torch.zeros_like(input_ids)
        x = self.ln_emb(self.word(input_ids) + self.position(pos) + self.token_type(tt))
        mask = token_mask = None
        if attention_mask is not None:
            mask = attention_mask[:, None, None, :].to(torch.bool)
            token_mask = attention_mask.to(torch.bool)
        for layer in self.layer:
            x = layer(x, mask, token_mask)
        logits = self.qa_outputs(x).float()
        start, end = logits[..., 0], logits[..., 1]
        if start_positions is None or end_positions is None:
            return start, end
        return 0.5 * (F.cross_entropy(start, start_positions) + F.cross_entropy(end, end_positions))

    def moe_layers(self):
        return [l.ffn for l in self.layer if l.is_moe]
