"""Expert-parallel checkpoints: per-rank shards with a manifest, and re-sharding to another EP degree.

Expert parameters are ordinary ``nn.Parameter`` tensors with the expert index first
(``experts.htoh4.weight [E_local, d_ffn, d_model]`` etc., mix_moe/mix_moe/transformer.py:32-36), so a rank's
``state_dict()`` holds only its own experts; the reference has no utility to gather or re-split them (its only
checkpoint code pickles a whole single-process model, mix_moe/mix_moe/examples/transformer-xl/train.py:524-531).
Because rank r owns experts [r * E_local, (r + 1) * E_local), re-sharding is a concatenation along dim 0
followed by an even split.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import torch
import torch.nn as nn


def expert_keys(model: nn.Module) -> List[str]:
    """state_dict keys of expert (non-replicated) parameters."""
    return [n for n, p in model.named_parameters() if getattr(p, "skip_allreduce", False)]


def ep_state_dict(model: nn.Module) -> Dict[str, Dict[str, torch.Tensor]]:
    """Split the model state into {'experts': local expert tensors, 'replicated': everything else} (on CPU)."""
    ek = set(expert_keys(model))
    sd = model.state_dict()
    return {"experts": {k: v.detach().cpu() for k, v in sd.items() if k in ek},
            "replicated": {k: v.detach().cpu() for k, v in sd.items() if k not in ek}}


def save_ep_checkpoint(model: nn.Module, prefix: str, ep_rank: int, ep_size: int, extra: Optional[dict] = None,
                       optimizer: Optional[torch.optim.Optimizer] = None):
    """Every rank writes ``<prefix>.ep<rank>of<size>.pt``; rank 0 also writes the replicated part and a manifest. With
    ``optimizer`` every rank also writes its optimizer state (``<prefix>.opt<rank>of<size>.pt``: it covers this rank's
    experts and its copy of the replicated parameters; it is reloaded only at the same expert-parallel degree)."""
    os.makedirs(os.path.dirname(os.path.abspath(prefix)) or ".", exist_ok=True)
    parts = ep_state_dict(model)
    torch.save(parts["experts"], f"{prefix}.ep{ep_rank}of{ep_size}.pt")
    if optimizer is not None:
        torch.save(optimizer.state_dict(), f"{prefix}.opt{ep_rank}of{ep_size}.pt")
    if ep_rank == 0:
        torch.save(parts["replicated"], f"{prefix}.replicated.pt")
        e_loc = {k: int(v.shape[0]) for k, v in parts["experts"].items()}
        with open(f"{prefix}.manifest.json", "w") as f:
            json.dump({"ep_size": ep_size, "experts_per_rank": e_loc, "expert_keys": sorted(parts["experts"]),
                       "extra": extra or {}}, f, indent=1)


def reshard_expert_state(shards: List[Dict[str, torch.Tensor]], new_ep_size: int) -> List[Dict[str, torch.Tensor]]:
    """shards[r] = expert tensors of old rank r -> list of ``new_ep_size`` dicts."""
    out: List[Dict[str, torch.Tensor]] = [dict() for _ in range(new_ep_size)]
    for k in shards[0]:
        full = torch.cat([s[k] for s in shards], 0)
        if full.shape[0] % new_ep_size:
            raise ValueError(f"{k}: {full.shape[0]} experts cannot be split over {new_ep_size} ranks")
        for r, piece in enumerate(torch.chunk(full, new_ep_size, 0)):
            out[r][k] = piece.clone()
    return out


def load_ep_checkpoint(model: nn.Module, prefix: str, ep_rank: int, ep_size: int, strict: bool = True,
                       optimizer: Optional[torch.optim.Optimizer] = None) -> dict:
    """Load a checkpoint written at any EP degree into a model sharded over ``ep_size`` ranks. ``optimizer`` state is
    restored when the checkpoint has it for this degree; after a change of degree the optimizer starts fresh (the
    returned manifest then carries ``"optimizer_restored": False``)."""
    with open(f"{prefix}.manifest.json") as f:
        manifest = json.load(f)
    old = int(manifest["ep_size"])
    if old == ep_size:
        experts = torch.load(f"{prefix}.ep{ep_rank}of{old}.pt", map_location="cpu")
    else:
        shards = [torch.load(f"{prefix}.ep{r}of{old}.pt", map_location="cpu") for r in range(old)]
        experts = reshard_expert_state(shards, ep_size)[ep_rank]
    state = dict(torch.load(f"{prefix}.replicated.pt", map_location="cpu"))
    state.update(experts)
    model.load_state_dict(state, strict=strict)
    if optimizer is not None:
        path = f"{prefix}.opt{ep_rank}of{ep_size}.pt"
        restored = old == ep_size and os.path.exists(path)
        if restored:
            optimizer.load_state_dict(torch.load(path, map_location="cpu"))
        manifest["optimizer_restored"] = restored
    return manifest


def import_reference_state(state: Dict[str, torch.Tensor], experts_per_rank: int) -> Dict[str, torch.Tensor]:
    """Adapt a ``state_dict`` written by the reference package. Its expert tensors carry three extra leading rows, the
    never-synchronised "popular expert" slots (``_Expert(num_local_expert + 3, ...)``,
    mix_moe/mix_moe/transformer.py:449-453); every tensor under an ``experts.`` key whose first dimension exceeds
    ``experts_per_rank`` is cut back to the real experts. Other entries are passed through."""
    out = {}
    for k, v in state.items():
        if ".experts." in "." + k and torch.is_tensor(v) and v.dim() >= 1 and v.shape[0] > experts_per_rank:
            v = v[:experts_per_rank].clone()
        out[k] = v
    return out
