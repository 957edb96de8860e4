"""Optimizers that run on the library's kernels."""
from __future__ import annotations

import ctypes as C

import torch

from .. import native as N

_BLOCK_ELEMS = 256 * 8 * 4      # elements one block of 256 threads covers in four passes of 16-byte vectors
_MAX_BLOCKS = 148 * 16


class FusedSGD(torch.optim.Optimizer):
    """Plain SGD (optional weight decay) for bf16 / fp16 CUDA parameters on csrc/moe_kernels.cu: full-width passes at the
    memory rate, up to 48 tensors per launch (``sgd_multi_kernel``), so that the hundreds of small tensors of a
    transformer (biases, LayerNorm weights, routers) cost a handful of launches instead of one each. Other parameters
    take the torch path. The reference's benchmark loops use torch.optim.SGD on half-precision parameters
    (mix_moe/mix_moe/examples/mix_moe_ddp.py:155)."""

    def __init__(self, params, lr: float = 1e-3, weight_decay: float = 0.0):
        super().__init__(params, dict(lr=lr, weight_decay=weight_decay))
        self._table = None

    @staticmethod
    def _eligible(p, g) -> bool:
        return (p.is_cuda and p.dtype in (torch.bfloat16, torch.float16) and g.dtype == p.dtype and p.is_contiguous()
                and g.is_contiguous() and p.data_ptr() % 16 == 0 and g.data_ptr() % 16 == 0 and p.numel() > 0)

    def _launch(self, lib, batch, lr, wd, fp16, stream):
        t = self._table
        if t is None:
            t = self._table = N.SgdMulti()
        first = 0
        for k, (p, g) in enumerate(batch):
            n = p.numel()
            t.p[k], t.g[k], t.n[k], t.first_block[k] = p.data_ptr(), g.data_ptr(), n, first
            first += max(1, min(_MAX_BLOCKS, (n + _BLOCK_ELEMS - 1) // _BLOCK_ELEMS))
        t.first_block[len(batch)] = first
        t.count, t.lr, t.wd, t.fp16 = len(batch), lr, wd, fp16
        N.check(lib.ccf_sgd_multi(C.byref(t), stream), "ccf_sgd_multi")
        N.count(1)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        lib = None
        for group in self.param_groups:
            lr, wd = float(group["lr"]), float(group["weight_decay"])
            batches = {}                      # (device, dtype) -> tensors waiting for one launch
            for p in group["params"]:
                g = p.grad
                if g is None:
                    continue
                if self._eligible(p, g):
                    key = (p.device, p.dtype)
                    batch = batches.setdefault(key, [])
                    batch.append((p, g))
                    if len(batch) == N.SGD_MULTI:
                        lib = lib or N.load()
                        with torch.cuda.device(p.device):
                            self._launch(lib, batch, lr, wd, int(p.dtype == torch.float16), N.stream_ptr())
                        batch.clear()
                else:
                    if wd:
                        g = g.add(p, alpha=wd)
                    p.add_(g, alpha=-lr)
            for (device, dtype), batch in batches.items():
                if batch:
                    lib = lib or N.load()
                    with torch.cuda.device(device):
                        self._launch(lib, batch, lr, wd, int(dtype == torch.float16), N.stream_ptr())
        return loss
