"""LayerNorm on the library's kernels (csrc/norm.cu) for half-precision CUDA activations.

``LayerNorm`` is a drop-in ``nn.LayerNorm`` (same parameters, same state-dict keys); inputs the kernels do not cover
(CPU, fp32, a normalised dimension above 2048 or not a multiple of 8, no affine parameters) take the torch path. The
models' transformer blocks normalise a ``[tokens, d_model]`` matrix twice each; forward and backward are one pass over
that matrix here, with the weight / bias gradients reduced in the same backward kernel.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import native as N

MAX_D = 2048


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        lib = N.load()
        d = x.shape[-1]
        x2 = x.reshape(-1, d).contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        w = weight.contiguous()
        b = None if bias is None else bias.contiguous()
        N.check(lib.ccf_layernorm_fwd(x2.data_ptr(), w.data_ptr(), N.ptr(b), y.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                      rows, d, float(eps), int(x.dtype == torch.float16), N.stream_ptr()), "ccf_layernorm_fwd")
        N.count(1)
        ctx.save_for_backward(x2, w, mean, rstd)
        ctx.has_bias = bias is not None
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        lib = N.load()
        x2, w, mean, rstd = ctx.saved_tensors
        rows, d = x2.shape
        dy2 = dy.reshape(rows, d).contiguous()
        dx = torch.empty_like(x2)
        dg = torch.zeros(d, dtype=torch.float32, device=x2.device)
        db = torch.zeros(d, dtype=torch.float32, device=x2.device) if ctx.has_bias else None
        N.check(lib.ccf_layernorm_bwd(x2.data_ptr(), dy2.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                      dx.data_ptr(), dg.data_ptr(), N.ptr(db), rows, d, int(x2.dtype == torch.float16),
                                      N.stream_ptr()), "ccf_layernorm_bwd")
        N.count(1)
        return dx.view(ctx.shape), dg.to(w.dtype), (db.to(w.dtype) if db is not None else None), None


def supported(x: torch.Tensor, normalized_shape, weight) -> bool:
    d = x.shape[-1] if x.dim() else 0
    return (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and weight is not None and weight.dtype == x.dtype
            and len(normalized_shape) == 1 and normalized_shape[0] == d and d % 8 == 0 and 8 <= d <= MAX_D and x.numel() > 0)


def layer_norm(x, normalized_shape, weight, bias, eps=1e-5):
    """``F.layer_norm`` that runs on the library's kernels where they apply."""
    if supported(x, tuple(normalized_shape), weight) and (bias is None or bias.dtype == x.dtype):
        return _LayerNormFn.apply(x, weight, bias, eps)
    return F.layer_norm(x, normalized_shape, weight, bias, eps)


class LayerNorm(nn.LayerNorm):
    """``nn.LayerNorm`` whose forward and backward run on csrc/norm.cu for bf16 / fp16 CUDA inputs."""

    def forward(self, x):
        return layer_norm(x, self.normalized_shape, self.weight, self.bias, self.eps)
