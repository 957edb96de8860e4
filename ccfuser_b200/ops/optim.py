"""Optimizers that run on the library's kernels."""
from __future__ import annotations

import torch

from .. import native as N


class FusedSGD(torch.optim.Optimizer):
    """Plain SGD (optional weight decay) for bf16 / fp16 CUDA parameters: one full-width pass per tensor
    (csrc/moe_kernels.cu: sgd_step_kernel). Other parameters take the torch path. The reference's benchmark loops
    use torch.optim.SGD on half-precision parameters (mix_moe/mix_moe/examples/mix_moe_ddp.py:155)."""

    def __init__(self, params, lr: float = 1e-3, weight_decay: float = 0.0):
        super().__init__(params, dict(lr=lr, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        lib = None
        for group in self.param_groups:
            lr, wd = float(group["lr"]), float(group["weight_decay"])
            for p in group["params"]:
                g = p.grad
                if g is None:
                    continue
                if (p.is_cuda and p.dtype in (torch.bfloat16, torch.float16) and g.dtype == p.dtype
                        and p.is_contiguous() and g.is_contiguous() and p.data_ptr() % 16 == 0 and g.data_ptr() % 16 == 0):
                    lib = lib or N.load()
                    N.check(lib.ccf_sgd_step(p.data_ptr(), g.data_ptr(), p.numel(), lr, wd,
                                             int(p.dtype == torch.float16), N.stream_ptr()), "ccf_sgd_step")
                    N.count(1)
                else:
                    if wd:
                        g = g.add(p, alpha=wd)
                    p.add_(g, alpha=-lr)
        return loss
