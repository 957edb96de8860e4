"""Router as one kernel: linear layer on the tensor cores with top-k + softmax in its epilogue (csrc/router.cu).

``fused_router(x, weight, bias, k)`` returns ``(idx [T, k] int32, w [T, k] fp32)`` like
``topk_softmax(F.linear(x, weight, bias), k)`` but without writing the logits, and with the selection made on fp32
accumulators (mix_moe/mix_moe/gates/naive_gate.py:31-38 is the computation). Backward: the gradient of the logits is
non-zero only in the k selected columns (``topk_softmax_bwd_kernel``); the two skinny products that follow
(``dlogits @ W`` and ``dlogits^T @ x``) are plain library GEMMs.

Selected with ``CCFUSER_FUSED_ROUTER=1``; the default router path is the library linear layer followed by the top-k
kernel.
"""
from __future__ import annotations

import torch

from .. import native as N
from .gemm import Workspace


class _FusedRouter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, k, want_logits):
        lib = N.load()
        t, d = x.shape
        e = weight.shape[0]
        if x.dtype not in (torch.bfloat16, torch.float16) or weight.dtype != x.dtype:
            raise TypeError("fused router: x and the router weight must both be bf16 or both fp16")
        x = x.contiguous()
        wt = weight.contiguous()
        b = None if bias is None else bias.to(x.dtype).contiguous()
        idx = torch.empty(t, k, dtype=torch.int32, device=x.device)
        w = torch.empty(t, k, dtype=torch.float32, device=x.device)
        logits = torch.empty(t, e, dtype=torch.float32, device=x.device) if want_logits else None
        ws = Workspace.get(x.device)
        dev = x.device.index if x.device.index is not None else torch.cuda.current_device()
        N.check(lib.ccf_router_topk(x.data_ptr(), wt.data_ptr(), N.ptr(b), t, d, e, k, int(x.dtype == torch.float16),
                                    idx.data_ptr(), w.data_ptr(), N.ptr(logits), ws.status.data_ptr(),
                                    5_000_000_000, dev, N.stream_ptr()), "ccf_router_topk")
        N.count(1)
        ctx.save_for_backward(x, wt, idx, w)
        ctx.has_bias = bias is not None
        ctx.mark_non_differentiable(idx)
        if want_logits:
            ctx.mark_non_differentiable(logits)
            return idx, w, logits
        return idx, w, None

    @staticmethod
    def backward(ctx, _gidx, gw, _glogits):
        lib = N.load()
        x, wt, idx, w = ctx.saved_tensors
        t, k = idx.shape
        e = wt.shape[0]
        dlogits = torch.zeros(t, e, dtype=x.dtype, device=x.device)
        gw = gw.contiguous().float()
        N.check(lib.ccf_topk_softmax_bwd(idx.data_ptr(), w.data_ptr(), gw.data_ptr(), t, e, k, dlogits.data_ptr(),
                                         int(x.dtype == torch.float16), 0, N.stream_ptr()), "ccf_topk_softmax_bwd")
        N.count(1)
        dx = dlogits @ wt if ctx.needs_input_grad[0] else None
        dw = dlogits.t() @ x if ctx.needs_input_grad[1] else None
        db = dlogits.sum(0) if (ctx.has_bias and ctx.needs_input_grad[2]) else None
        return dx, dw, db, None, None


def fused_router(x: torch.Tensor, weight: torch.Tensor, bias, k: int, want_logits: bool = False):
    """-> (idx, w) or, with ``want_logits``, (idx, w, fp32 logits; not differentiable)."""
    idx, w, logits = _FusedRouter.apply(x, weight, bias, k, want_logits)
    return (idx, w, logits) if want_logits else (idx, w)


def supported(x: torch.Tensor, weight: torch.Tensor, k: int) -> bool:
    t, d = x.shape
    e = weight.shape[0]
    return (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and weight.dtype == x.dtype and t >= 1
            and e <= 256 and 1 <= k <= min(8, e) and d >= 64 and d % 8 == 0)
