"""Configuration of one expert-parallel MoE FFN layer.

The reference hard-codes most of these knobs (block size 64 at
mix_moe/mix_moe/layers.py:66, top-2 buffer factor at mix_moe/csrc/mix_moe.h:77,
fp16 only at mix_moe/csrc/mix_moe.h:242-245, GELU at mix_moe/mix_moe/transformer.py:445);
here they are one frozen dataclass that every backend reads.
"""
from __future__ import annotations

import dataclasses
import math
import os
from typing import Optional

import torch

ACTIVATIONS = ("gelu", "relu", "swiglu")
BACKENDS = ("auto", "fused", "nccl", "cpu")


@dataclasses.dataclass(frozen=True)
class MoEConfig:
    """Static description of an MoE FFN layer.

    d_model / d_ffn      feature sizes of the expert FFN (d_model -> d_ffn -> d_model)
    num_experts          total number of experts over the expert-parallel group
    top_k                experts chosen per token
    capacity_factor      >0: each (source rank, expert) pair keeps at most
                         ceil(capacity_factor * tokens * top_k / num_experts) routed rows,
                         later rows (in token-major slot order) are dropped;
                         0 or None: nothing is dropped
    activation           'gelu' | 'relu' | 'swiglu' (swiglu adds a second up projection)
    bias                 expert linear layers carry a bias (the reference always does)
    dtype                parameter / compute dtype
    ep_size              expert-parallel world size (experts are split evenly)
    backend              'fused' (sm_100a kernels), 'nccl' (all_to_all_single + library GEMM
                         baseline), 'cpu' (same code path over gloo), 'auto'
    max_tokens           upper bound of tokens per rank per call; sizes the symmetric buffers
    recv_factor          without a capacity factor the receive buffer of a rank is sized
                         recv_factor x the balanced load (overflow is reported, not silent)
    router_dtype         parameter / compute dtype of the router's linear layer; None = ``dtype``. torch.float32 keeps
                         the routing decisions independent of half-precision rounding of the logits
    aux_loss_coef        weight of the router's load-balance loss (0 = off); z_loss_coef: weight of its z-loss.
                         The layer's gate records their sum for the training loop (gate.get_loss())
    shared_ffn           >0: hidden size of an always-on dense FFN (same activation as the experts) whose output is added
                         to the routed experts' output for every token; its parameters are replicated like the router's
    shadow_experts       >0: the n most popular experts of every step are replicated to all ranks for that step
                         (weights broadcast, gradients reduced back to the owner) and their tokens are computed
                         where they are; see parallel/shadow.py
    """

    d_model: int
    d_ffn: int
    num_experts: int
    top_k: int = 2
    capacity_factor: Optional[float] = None
    activation: str = "gelu"
    bias: bool = True
    dtype: torch.dtype = torch.bfloat16
    ep_size: int = 1
    backend: str = "auto"
    max_tokens: int = 4096
    recv_factor: float = 2.0
    router_bias: bool = True
    shadow_experts: int = 0
    router_dtype: Optional[torch.dtype] = None
    aux_loss_coef: float = 0.0
    z_loss_coef: float = 0.0
    shared_ffn: int = 0

    def __post_init__(self):
        if self.activation not in ACTIVATIONS:
            raise ValueError(f"activation must be one of {ACTIVATIONS}, got {self.activation!r}")
        if self.backend not in BACKENDS:
            raise ValueError(f"backend must be one of {BACKENDS}, got {self.backend!r}")
        if self.num_experts % self.ep_size != 0:
            raise ValueError("num_experts must be divisible by ep_size")
        if not (1 <= self.top_k <= self.num_experts):
            raise ValueError("top_k must be in [1, num_experts]")
        if not (0 <= self.shadow_experts <= self.num_experts):
            raise ValueError("shadow_experts must be in [0, num_experts]")

    @property
    def experts_per_rank(self) -> int:
        return self.num_experts // self.ep_size

    def capacity(self, tokens: int) -> int:
        """Rows one source rank may send to one expert for a call with `tokens` tokens."""
        slots = tokens * self.top_k
        if not self.capacity_factor or self.capacity_factor <= 0:
            return slots
        return min(slots, int(math.ceil(self.capacity_factor * slots / self.num_experts)))

    def max_recv_rows(self, tokens: Optional[int] = None, tile: int = 128) -> int:
        """Upper bound of rows (tile padded, per expert) a rank must be able to receive."""
        tokens = self.max_tokens if tokens is None else tokens
        e_loc = self.experts_per_rank
        if self.capacity_factor and self.capacity_factor > 0:
            per_expert = self.ep_size * self.capacity(tokens)
            per_expert = (per_expert + tile - 1) // tile * tile
            return e_loc * per_expert
        balanced = tokens * self.top_k  # == ep_size * tokens * top_k / ep_size
        rows = int(math.ceil(self.recv_factor * balanced)) + e_loc * tile
        rows = min(rows, self.ep_size * tokens * self.top_k + e_loc * tile)
        return (rows + tile - 1) // tile * tile

    def memory_estimate(self, layers: int = 1, training: bool = True) -> dict:
        """Device memory per rank, in bytes, of ``layers`` fused MoE layers of this configuration that share one
        expert-parallel group: parameters (and their gradients), the per-layer receive / combine / activation buffers,
        the buffers shared by the layers of a group, and the transient tensors of one backward pass. For sizing
        ``max_tokens`` and ``recv_factor`` against the 180 GB of a B200."""
        esz = 2 if self.dtype in (torch.bfloat16, torch.float16) else 4
        e_loc, d, f = self.experts_per_rank, self.d_model, self.d_ffn
        mats = 3 if self.activation == "swiglu" else 2
        rows, slots = self.max_recv_rows(), self.max_tokens * self.top_k
        weights = e_loc * (mats * d * f + ((mats - 1) * f + d if self.bias else 0)) * esz
        rsz = 4 if self.router_dtype == torch.float32 else esz
        router = self.num_experts * (d + (1 if self.router_bias else 0)) * rsz
        if self.shared_ffn > 0:      # counted with the router: replicated, small next to the experts
            router += (mats * d * self.shared_ffn + ((mats - 1) * self.shared_ffn + d if self.bias else 0)) * esz
        per_layer = (rows * d + slots * d) * esz                                   # xrecv + comb (symmetric)
        per_layer += rows * f * esz * (mats if training else 1)                    # h_act (+ pre-activations)
        per_layer += (3 * slots + 2 * self.num_experts + 6 * e_loc) * 4            # routing index arrays
        shared = (rows * d + slots * d) * esz + rows * 8                           # grecv + gcomb + row metadata
        transient = (rows * f * esz * (mats - 1) + weights) if training else 0     # dh(, dh2) + weight gradients of one layer
        out = {"parameters": layers * (weights + router), "gradients": layers * (weights + router) if training else 0,
               "layer_buffers": layers * per_layer, "group_buffers": shared, "backward_transient": transient}
        out["total"] = sum(out.values())
        return out

    def replace(self, **kw) -> "MoEConfig":
        return dataclasses.replace(self, **kw)


def env_flag(name: str, default: int = 0) -> int:
    """Integer debug switch read from the environment (CCFUSER_<NAME>)."""
    try:
        return int(os.environ.get("CCFUSER_" + name, default))
    except ValueError:
        return default
