"""The user-facing MoE FFN layer.

``MoELayer`` is the new API; ``MixMOETransformerMLP`` / ``MixMOE`` keep the constructor of the reference
(mix_moe/mix_moe/transformer.py:428-448, mix_moe/mix_moe/layers.py:33-60) so its users can switch over.
Forward semantics follow mix_moe/mix_moe/transformer.py:475-497 and layers.py:550-568: flatten to
``[T, d_model]``, route top-k, run each kept (token, slot) through its expert, sum the slots weighted by the
gate scores, reshape back. Planning is done on the device; there is no Python planner thread
(transformer.py:102-426).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .config import MoEConfig
from .experts import Experts, scan_expert_params
from .gates import NaiveGate
from .parallel.a2a import moe_forward_a2a
from .parallel.placement import placement_cost, plan_placement, rebalance_experts
from .parallel.shadow import ShadowFused, gather_shadow_params, select_popular, shadow_forward, split_shadow_slots


class MoELayer(nn.Module):
    """Expert-parallel MoE FFN: ``y = sum_j keep_j * g_j * FFN_{e_j}(x)``.

    Parameters live under ``gate.gate.{weight,bias}`` and ``experts.{htoh4,h4toh}.{weight,bias}``
    (plus ``experts.htoh4_gate.*`` for SwiGLU). Each rank of ``ep_group`` owns
    ``num_experts / ep_size`` consecutive experts (mix_moe/mix_moe/transformer.py:120-122).
    """

    def __init__(self, config: MoEConfig, ep_group=None, device=None, gate: Optional[nn.Module] = None):
        super().__init__()
        self.config = config
        if ep_group is None and dist.is_initialized() and config.ep_size > 1:
            ep_group = dist.group.WORLD
        self.ep_group = ep_group
        world = dist.get_world_size(ep_group) if (dist.is_initialized() and config.ep_size > 1) else 1
        if world != config.ep_size:
            raise ValueError(f"config.ep_size={config.ep_size} but the expert-parallel group has {world} ranks")
        self.ep_rank = dist.get_rank(ep_group) if world > 1 else 0
        e_loc = config.experts_per_rank
        self.gate = gate if gate is not None else NaiveGate(
            config.d_model, e_loc, config.ep_size, config.top_k, bias=config.router_bias,
            aux_loss_coef=config.aux_loss_coef, z_loss_coef=config.z_loss_coef)
        self.gate.to(device=device, dtype=config.router_dtype or config.dtype)
        self.experts = Experts(e_loc, config.d_model, config.d_ffn, config.activation, config.bias,
                               dtype=config.dtype, device=device)
        scan_expert_params(self.experts)
        for p in self.gate.parameters():
            setattr(p, "dp_comm", "gate")
        # optional always-on dense FFN next to the routed experts ("shared expert"): replicated parameters, library GEMMs
        self.shared = None
        if config.shared_ffn > 0:
            self.shared = Experts(1, config.d_model, config.shared_ffn, config.activation, config.bias,
                                  dtype=config.dtype, device=device)
        self._fused = None
        self._shadow_fused = None
        self._sgd = None
        self.last_stats = {}

    # ---- backend selection -------------------------------------------------------------------
    def backend(self, x: torch.Tensor) -> str:
        b = self.config.backend
        if b == "auto":
            return "fused" if x.is_cuda else "cpu"
        return b

    def _fused_impl(self):
        if self._fused is None:
            from .ops.fused import FusedMoE  # needs the CUDA library
            self._fused = FusedMoE(self)
            self._fused.sgd = self._sgd
        return self._fused

    # ---- forward -----------------------------------------------------------------------------
    def forward(self, inp: torch.Tensor, token_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``inp [..., d_model]``. ``token_mask`` (bool, shape ``inp.shape[:-1]``, True = real token): tokens marked
        False (padding) are not routed at all: they cost no expert compute, take no capacity, cross no link, and their
        output rows are zero. Stays on the device (no host synchronisation)."""
        cfg = self.config
        shape = inp.shape
        x = inp.reshape(-1, cfg.d_model)
        backend = self.backend(x)
        group = self.ep_group if cfg.ep_size > 1 else None
        if backend == "fused":
            fused = self._fused_impl()
            x = x.contiguous()
            idx, score = fused.route(x)
        else:
            idx, score = self.gate(x)
        if token_mask is not None:
            keep = token_mask.reshape(-1, 1).to(device=idx.device, dtype=torch.bool)
            idx = torch.where(keep, idx, torch.full_like(idx, -1))
        y_shadow = None
        if cfg.shadow_experts > 0:
            # the step's most popular experts are replicated: their slots leave the expert-parallel path
            shadow_ids = select_popular(idx, cfg.num_experts, cfg.shadow_experts, group)
            params = gather_shadow_params(self.experts, shadow_ids, self.ep_rank, group)
            idx, which = split_shadow_slots(idx, shadow_ids)
            if backend == "fused":
                if self._shadow_fused is None:
                    self._shadow_fused = ShadowFused(self, cfg.shadow_experts)
                y_shadow = self._shadow_fused(x, which, score, params, cfg.activation)
            else:
                y_shadow = shadow_forward(x, which, score, params, cfg.activation)
            self.last_stats["shadow_ids"] = shadow_ids
        if backend == "fused":
            y = fused.run_experts(x, idx, score)
        else:
            y = moe_forward_a2a(x, idx, score, self.experts, num_experts=cfg.num_experts,
                                capacity=cfg.capacity(x.shape[0]), group=group, stats=self.last_stats)
            y = y.to(inp.dtype)
        if y_shadow is not None:
            y = y + y_shadow.to(y.dtype)
        if self.shared is not None:
            y = y + self.shared.expert_forward(0, x).to(y.dtype)
        return y.reshape(shape[:-1] + (y.shape[-1],))

    # ---- placement ---------------------------------------------------------------------------
    def count_table(self) -> Optional[torch.Tensor]:
        """``[source rank, expert]`` kept rows of the last forward call (identical on every rank), or None before the
        first call. Reading it on the host synchronises; meant for the occasional placement decision."""
        if self._fused is not None:
            return self._fused.routing_stats()["count_table"]
        return self.last_stats.get("count_table")

    def rebalance(self, placement=None, optimizer=None, topology=None, slack: float = 0.05, min_gain: float = 0.0):
        """Move experts between ranks (collective over the expert-parallel group). With ``placement=None`` a placement
        is planned from the counts of the last forward call; see parallel/placement.py. A planned placement is applied
        only if it lowers the load of the busiest rank by at least the fraction ``min_gain`` (every rank takes the same
        decision from the same table), so a periodic call does not shuffle weights for nothing. Returns the placement
        used (the identity when nothing moved)."""
        identity = list(range(self.config.num_experts))
        if placement is None:
            table = self.count_table()
            if table is None:
                raise RuntimeError("no routing counts yet: run a forward pass first or pass a placement")
            e_loc = self.config.experts_per_rank
            placement = plan_placement(table, e_loc, topology, slack)
            before = placement_cost(table, identity, e_loc)["max_rank_rows"]
            after = placement_cost(table, placement, e_loc)["max_rank_rows"]
            if before <= 0 or (before - after) / before < min_gain or after >= before:
                return identity
        rebalance_experts(self, placement, optimizer)
        return list(placement)

    def fuse_sgd(self, lr: Optional[float], weight_decay: float = 0.0):
        """Apply plain SGD to the expert weight matrices inside the backward pass: the weight-gradient GEMMs' epilogue
        writes ``w - lr * (dw + weight_decay * w)`` over ``w`` instead of storing ``dw``, so the gradient is never
        written and the optimizer never reads it and the weights again (with many experts per GPU that traffic is a
        large part of a step). The matrices' ``.grad`` stays ``None`` (an optimizer skips them); biases and the router
        keep the ordinary path. Same update as ``torch.optim.SGD`` without momentum, computed from the fp32 accumulator.
        On a single-rank layer (``ep_size == 1``) every expert matrix is updated this way. On a layer that spans ranks
        only the second projection (``h4toh``) is: the first projection is still read by the input-gradient GEMM, which
        with peers has to stay the last kernel of a backward pass, so it keeps its gradient and the optimizer's update.
        For the fused backend; not compatible with gradient accumulation, clipping, replicated (shadow) experts or
        anything else that needs the expert weight gradients. ``lr=None`` switches it off. Call it again whenever the
        learning rate changes."""
        if lr is None:
            if self._fused is not None:
                self._fused.sgd = None
            self._sgd = None
            return
        if getattr(self.config, "shadow_experts", 0) > 0:
            raise ValueError("fuse_sgd is not available with shadow_experts > 0: the replicas return weight gradients to "
                             "the experts' owners")
        self._sgd = (float(lr), float(weight_decay))
        if self._fused is not None:
            self._fused.sgd = self._sgd

    def routing_stats(self):
        """Statistics of the last fused forward call as device tensors (see FusedMoE.routing_stats)."""
        return self._fused.routing_stats() if self._fused is not None else {}

    def check_status(self):
        """Host read of the fused kernels' status word; raises MoECommTimeout / MoEOverflow / MoECommError. With
        CCFUSER_CANARY=1 the guard regions around the symmetric buffers are verified as well."""
        if self._fused is not None:
            self._fused.ctx.check_status("MoELayer")
            if self._fused.ctx.guard:
                self._fused.ctx.check_canaries(extra=(self._fused.buf,))

    def release(self):
        """Free the symmetric buffers of the fused path (collective)."""
        if self._shadow_fused is not None:
            self._shadow_fused.close()
            self._shadow_fused = None
        if self._fused is not None:
            self._fused.close()
            self._fused = None

    def extra_repr(self):
        c = self.config
        extra = ""
        if c.shadow_experts:
            extra += f", shadow_experts={c.shadow_experts}"
        if c.shared_ffn:
            extra += f", shared_ffn={c.shared_ffn}"
        if c.router_dtype is not None:
            extra += f", router_dtype={c.router_dtype}"
        return (f"experts={c.num_experts} (local {c.experts_per_rank}), top_k={c.top_k}, d_model={c.d_model}, "
                f"d_ffn={c.d_ffn}, act={c.activation}, capacity_factor={c.capacity_factor}, backend={c.backend}{extra}")


class MixMOE(MoELayer):
    """Constructor-compatible stand-in for the reference base class (mix_moe/mix_moe/layers.py:33-60)."""

    def __init__(self, num_expert=32, d_model=1024, world_size=1, top_k=2, gate=NaiveGate,
                 d_hidden=4096, activation="gelu", moe_group=None, capacity_factor=None,
                 dtype=torch.float32, backend="auto", max_tokens=4096, device=None):
        cfg = MoEConfig(d_model=d_model, d_ffn=d_hidden, num_experts=num_expert * world_size, top_k=top_k,
                        capacity_factor=capacity_factor, activation=_act_name(activation), dtype=dtype,
                        ep_size=world_size, backend=backend, max_tokens=max_tokens)
        gate_mod = gate(d_model, num_expert, world_size, top_k) if isinstance(gate, type) else gate
        super().__init__(cfg, ep_group=moe_group, device=device, gate=gate_mod)
        self.num_expert, self.d_model, self.world_size, self.top_k = num_expert, d_model, world_size, top_k

    def mark_parallel_comm(self, expert_dp_comm="none"):
        """FastMoE-style communication tags (mix_moe/mix_moe/layers.py:70-83)."""
        for p in self.experts.parameters():
            setattr(p, "dp_comm", expert_dp_comm)
        for p in self.gate.parameters():
            setattr(p, "dp_comm", "gate")


class MixMOETransformerMLP(MixMOE):
    """``MixMOETransformerMLP(gate_type, experts, model_dim, expert_rank, world_size, ...)`` as in
    mix_moe/mix_moe/transformer.py:435-448. ``experts`` is the reference's dict: ``num_local_expert`` (experts per
    rank) and ``hidden_size`` (FFN width) as read at transformer.py:449-450 and passed by
    examples/mix_moe_ddp.py:109, with the optional ``activation_fn``; Tutel's spelling of the same two entries
    (``count_per_node``, ``hidden_size_per_expert``) is accepted as well. Both entries are required: a missing one
    raises instead of silently building one expert of width 4 * model_dim. Unlike the reference the activation named
    there is honoured (``'gelu' | 'relu' | 'swiglu'`` or an nn.Module)."""

    def __init__(self, gate_type=None, experts=None, model_dim=1024, expert_rank=0, world_size=1,
                 scan_expert_func=None, total_batch_size=4096, expert_dp_comm="none",
                 activation=None, top_k=None, moe_group=None, capacity_factor=None,
                 dtype=torch.float32, backend="auto", device=None):
        experts = experts or {}
        gate_type = gate_type or {}
        k = top_k if top_k is not None else gate_type.get("k", 2)
        act = activation if activation is not None else experts.get("activation_fn", "gelu")

        def entry(*names):
            for n in names:
                if n in experts:
                    return int(experts[n])
            raise KeyError(f"experts dict needs {names[0]!r} (or {names[1]!r}); got keys {sorted(experts)}")

        super().__init__(num_expert=entry("num_local_expert", "count_per_node"), d_model=model_dim,
                         world_size=world_size, top_k=k, d_hidden=entry("hidden_size", "hidden_size_per_expert"),
                         activation=act, moe_group=moe_group,
                         capacity_factor=capacity_factor if capacity_factor is not None else gate_type.get("capacity_factor"),
                         dtype=dtype, backend=backend, max_tokens=total_batch_size, device=device)
        if scan_expert_func is not None:
            for n, p in self.experts.named_parameters():
                scan_expert_func(n, p)
        self.mark_parallel_comm(expert_dp_comm)

    def async_expert_assignment(self, x):
        """Kept as a no-op: routing and planning run on the device inside ``forward``, so there is
        nothing to overlap on a host thread (mix_moe/mix_moe/transformer.py:463-466)."""
        return None


def _act_name(a) -> str:
    if isinstance(a, str):
        return a.lower()
    if isinstance(a, nn.GELU) or a is torch.nn.functional.gelu:
        return "gelu"
    if isinstance(a, nn.ReLU) or a is torch.nn.functional.relu:
        return "relu"
    if a is None:
        return "gelu"
    raise ValueError(f"unsupported expert activation {a!r} (use 'gelu', 'relu' or 'swiglu')")
