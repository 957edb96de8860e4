"""Expert parameters with the reference's state-dict layout.

Keys and shapes (mix_moe/mix_moe/transformer.py:32-36,78-79): ``htoh4.weight [E_local, d_ffn, d_model]``,
``htoh4.bias [E_local, d_ffn]``, ``h4toh.weight [E_local, d_model, d_ffn]``, ``h4toh.bias [E_local, d_model]``
(``[expert, out, in]``, the nn.Linear convention). SwiGLU experts add ``htoh4_gate.*`` with the shape of
``htoh4.*``; it has no counterpart in the reference. The kernels read these tensors in place: the
``[out, in]`` layout is K-major for ``x @ W.T`` and is described directly to the tensor cores, instead of
the per-call ``transpose().contiguous()`` of mix_moe/mix_moe/linear.py:74,130.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class ExpertLinear(nn.Module):
    """A stack of ``num_expert`` independent linear layers."""

    def __init__(self, num_expert: int, in_feat: int, out_feat: int, bias: bool = True,
                 dtype=None, device=None):
        super().__init__()
        self.num_expert, self.in_feat, self.out_feat = num_expert, in_feat, out_feat
        self.weight = nn.Parameter(torch.empty(num_expert, out_feat, in_feat, dtype=dtype, device=device))
        if bias:
            self.bias = nn.Parameter(torch.zeros(num_expert, out_feat, dtype=dtype, device=device))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self):
        # per-expert nn.Linear initialisation (the reference applies kaiming_uniform_(a=sqrt(5)) to the
        # 3-D weight as a whole and also to the bias, transformer.py:63-65; the per-expert fan-in is used here)
        bound = 1.0 / math.sqrt(self.in_feat)
        with torch.no_grad():
            self.weight.uniform_(-bound, bound)
            if self.bias is not None:
                self.bias.uniform_(-bound, bound)

    def extra_repr(self):
        return f"num_expert={self.num_expert}, in={self.in_feat}, out={self.out_feat}, bias={self.bias is not None}"


class Experts(nn.Module):
    """``E_local`` FFN experts: htoh4 -> activation -> h4toh."""

    def __init__(self, num_expert: int, d_model: int, d_ffn: int, activation: str = "gelu",
                 bias: bool = True, dtype=None, device=None):
        super().__init__()
        self.activation = activation
        self.htoh4 = ExpertLinear(num_expert, d_model, d_ffn, bias, dtype, device)
        if activation == "swiglu":
            self.htoh4_gate = ExpertLinear(num_expert, d_model, d_ffn, bias, dtype, device)
        self.h4toh = ExpertLinear(num_expert, d_ffn, d_model, bias, dtype, device)

    def expert_forward(self, e: int, x: torch.Tensor) -> torch.Tensor:
        """Plain torch forward of local expert ``e`` on rows ``x`` (oracle and library backends)."""
        b1 = self.htoh4.bias[e] if self.htoh4.bias is not None else None
        h = F.linear(x, self.htoh4.weight[e], b1)
        if self.activation == "swiglu":
            bg = self.htoh4_gate.bias[e] if self.htoh4_gate.bias is not None else None
            g = F.linear(x, self.htoh4_gate.weight[e], bg)
            h = F.silu(g) * h
        elif self.activation == "gelu":
            h = F.gelu(h)
        else:
            h = F.relu(h)
        b2 = self.h4toh.bias[e] if self.h4toh.bias is not None else None
        return F.linear(h, self.h4toh.weight[e], b2)


def scan_expert_params(module: nn.Module):
    """Tag every expert parameter so data-parallel wrappers leave it alone
    (the ``skip_allreduce`` convention of mix_moe/mix_moe/transformer.py:454-456)."""
    for _, p in module.named_parameters():
        setattr(p, "skip_allreduce", True)
        setattr(p, "dp_comm", "none")
