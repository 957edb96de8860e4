"""Router as one kernel: linear layer on the tensor cores with top-k + softmax in its epilogue (csrc/router.cu).

``fused_router(x, weight, bias, k)`` returns ``(idx [T, k] int32, w [T, k] fp32)`` like
``topk_softmax(F.linear(x, weight, bias), k)`` but without writing the logits, and with the selection made on fp32
accumulators (mix_moe/mix_moe/gates/naive_gate.py:31-38 is the computation).

Backward uses no library GEMM either. The gradient of the logits that comes from the gate weights is non-zero only in
the k selected columns, so ``dx`` is a weighted sum of k router rows per token and ``dW`` a scatter-add of scaled token
rows (``router_bwd_dx_kernel`` / ``router_bwd_dw_kernel``): both read or write one ``[T, d]`` matrix once. When the
fp32 logits are requested as a differentiable output (auxiliary router losses), their dense gradient is added and the
two products run on this library's own tcgen05 grouped GEMM (ops/gemm.py), padded to its tile sizes.

This is the default router of the fused backend whenever ``supported`` holds (``CCFUSER_FUSED_ROUTER=0`` selects the
library linear layer followed by the top-k kernel, which is also what a router kept in fp32 next to half-precision
experts uses).
"""
from __future__ import annotations

import torch

from .. import native as N
from . import gemm as G
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
            return idx, w, logits
        return idx, w, None

    @staticmethod
    def backward(ctx, _gidx, gw, glogits):
        lib = N.load()
        x, wt, idx, w = ctx.saved_tensors
        t, k = idx.shape
        e, d = wt.shape
        fp16 = int(x.dtype == torch.float16)
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        need_b = ctx.has_bias and ctx.needs_input_grad[2]
        gw = torch.zeros_like(w) if gw is None else gw.contiguous().float()
        if glogits is None:
            # only the k selected columns carry a gradient: dx needs no [T, E] matrix and no GEMM
            dx = torch.empty_like(x) if need_x else None
            big = t >= 4096 and (need_w or need_b)
            dw32 = torch.zeros(e, d, dtype=torch.float32, device=x.device) if ((need_w or need_b) and not big) else None
            db32 = torch.zeros(e, dtype=torch.float32, device=x.device) if (need_b and not big) else None
            if dx is not None or dw32 is not None:
                N.check(lib.ccf_router_bwd(idx.data_ptr(), w.data_ptr(), gw.data_ptr(), wt.data_ptr(), x.data_ptr(), N.ptr(dx),
                                           N.ptr(dw32), N.ptr(db32), t, d, e, k, fp16, N.stream_ptr()), "ccf_router_bwd")
                N.count(int(need_x) + int(dw32 is not None))
            if not big:
                return (dx, dw32.to(wt.dtype) if need_w else None, db32.to(wt.dtype) if need_b else None, None, None)
            # many tokens: the scatter-add of token rows into E weight rows is a [E, T] x [T, d] product with a sparse
            # left factor; on the tensor cores (own grouped GEMM, reduction over the tokens) it beats atomics
            ep = 128 if e <= 128 else 256
            dlp = torch.zeros(t, ep, dtype=x.dtype, device=x.device)
            N.check(lib.ccf_topk_softmax_bwd(idx.data_ptr(), w.data_ptr(), gw.data_ptr(), t, ep, k, dlp.data_ptr(), fp16, 0,
                                             N.stream_ptr()), "ccf_topk_softmax_bwd")
            N.count(1)
            dw = _dw_by_gemm(dlp, x, e, d, wt.dtype) if need_w else None
            db = dlp[:, :e].float().sum(0).to(wt.dtype) if need_b else None
            return dx, dw, db, None, None
        # dense gradient of the logits (auxiliary losses) + the selected columns' part, then two products on the
        # tcgen05 grouped GEMM: [T, Ep] x [Ep, d] and [Ep, T] x [T, d], Ep = E padded to the 128-row tile
        dl = torch.zeros(t, e, dtype=torch.float32, device=x.device)
        N.check(lib.ccf_topk_softmax_bwd(idx.data_ptr(), w.data_ptr(), gw.data_ptr(), t, e, k, dl.data_ptr(), 0, 1,
                                         N.stream_ptr()), "ccf_topk_softmax_bwd")
        N.count(1)
        dl = dl + glogits.float()
        ep = 128 if e <= 128 else 256
        dlp = torch.zeros(t, ep, dtype=x.dtype, device=x.device)
        dlp[:, :e] = dl
        gb, gr = G.single_group(t, x.device)
        dx = dw = None
        if need_x:
            dx = torch.empty_like(x)
            G.launch(a0=dlp, b0=wt, a_major=N.MAJ_K, b_major=N.MAJ_MN, epi=N.EPI_STORE, n=d, k=ep, group_base=gb,
                     group_rows=gr, num_groups=1, b_group_rows=0, out0=dx)
        if need_w:
            dw = _dw_by_gemm(dlp, x, e, d, wt.dtype)
        db = dl.sum(0).to(wt.dtype) if need_b else None
        return dx, dw, db, None, None


def _dw_by_gemm(dlp: torch.Tensor, x: torch.Tensor, e: int, d: int, dtype) -> torch.Tensor:
    """dW [e, d] = dlp[:, :e]^T x on the library's k-grouped GEMM; ``dlp [T, 128 or 256]`` is the logits' gradient,
    zero-padded to the kernel's tile height. The token range is cut into up to 16 groups, each reduced by its own
    tiles (one group alone would occupy d / 256 CTAs for the whole reduction), and the partial sums are added."""
    t, ep = dlp.shape
    groups = max(1, min(16, t // 1024))
    per = (t + groups - 1) // groups
    per = (per + 127) // 128 * 128
    base = torch.arange(groups, dtype=torch.int32, device=x.device) * per
    rows = (t - base).clamp(min=0, max=per).to(torch.int32)
    dwp = torch.empty(groups, ep, d, dtype=torch.float32, device=x.device)
    G.launch(a0=dlp, b0=x, a_major=N.MAJ_MN, b_major=N.MAJ_MN, epi=N.EPI_STORE, n=d, kgroup=True, m_per_group=ep,
             group_base=base, group_rows=rows, num_groups=groups, out0=dwp, ld_out=d, out_fp32=True)
    return dwp[:, :e].sum(0).to(dtype)


def fused_router(x: torch.Tensor, weight: torch.Tensor, bias, k: int, want_logits: bool = False):
    """-> (idx, w) or, with ``want_logits``, (idx, w, fp32 logits). The logits are differentiable: a loss computed from
    them (load balance, z-loss) sends its gradient back to x and the router parameters."""
    idx, w, logits = _FusedRouter.apply(x, weight, bias, k, want_logits)
    return (idx, w, logits) if want_logits else (idx, w)


def supported(x: torch.Tensor, weight: torch.Tensor, k: int) -> bool:
    t, d = x.shape
    e = weight.shape[0]
    return (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and weight.dtype == x.dtype and t >= 1
            and e <= 256 and 1 <= k <= min(8, e) and d >= 64 and d % 32 == 0)
