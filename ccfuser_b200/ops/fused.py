"""The fused expert-parallel forward and backward of one MoE FFN layer on sm_100a.

Per call, on every rank (nothing touches the host, nothing calls a library collective):

    route        top-k softmax kernel -> deterministic positions and kept counts per expert
    plan         kept counts are stored into every rank's count table (peer stores + epoch flag); each
                 rank derives the dense row layout of every owner's receive buffer
    GEMM-1       ONE kernel: its first CTAs push this rank's routed rows into the owners' receive buffers
                 (peer stores, per-128-row-tile arrival counters); all CTAs then run tcgen05 tiles, each
                 tile starting as soon as its rows have landed; epilogue = bias + activation
    GEMM-2       tcgen05 tiles; the epilogue adds the bias, multiplies by the gate weight and stores each
                 row into the combine buffer of the rank the token came from, then bumps that rank's
                 completion counter
    reduce       the source waits for its counters and sums the k slots of every token

Backward mirrors it: g*dy rows are pushed (same kernel as dgrad-2, whose epilogue applies the activation
derivative), wgrad-2 / wgrad-1 reduce over the saved rows with MN-major operands, dgrad-1's epilogue
stores dx rows into the source's buffer.

Call stack being replaced: mix_moe/mix_moe/linear.py:60-173 (MixMOELinear1/2 autograd functions) ->
mix_moe/csrc/mix_moe.h:236-505 (first/second_gemm_forward/backward) -> mix_moe/csrc/cuda/mix_gemm.cu.
Buffer hazards between calls are covered by the completion counters: a rank cannot start the dispatch of
call i+1 before every owner has finished the last kernel of call i, so one receive buffer per role is
enough (the reference aliases one buffer for everything and separates uses with global barriers,
mix_moe/csrc/mix_moe.h:271,336,420,467).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict

import torch

from .. import native as N
from ..config import env_flag
from ..gates import router_aux_loss
from ..parallel.symm import SymmBuffer
from ..utils.tracing import nvtx_range
from . import gemm as G
from . import router as R

TILE = 128


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class CommContext:
    """Symmetric state shared by all fused layers of one expert-parallel group: backward receive and
    combine buffers, row metadata, tile arrival counters, the count table and the completion counters."""

    _instances: Dict[tuple, "CommContext"] = {}

    def __init__(self, group, world, rank, device, max_rows, max_slots, d_model, e_total, dtype):
        self.group, self.world, self.rank, self.device = group, world, rank, device
        self.max_rows, self.max_slots, self.d_model, self.e_total, self.dtype = max_rows, max_slots, d_model, e_total, dtype
        esz = 2
        sizes = {
            "grecv": max_rows * d_model * esz,
            "gcomb": max_slots * d_model * esz,
            "row_src": max_rows * 4,
            "row_gate": max_rows * 4,
            "tile_flags": (max_rows // TILE + 1) * 4,
            "cnt_table": world * e_total * 4,
            "cnt_flag": N.MAX_RANKS * 4,
            "done": N.MAX_RANKS * 4,
            "bar_flag": N.MAX_RANKS * 4,
        }
        # CCFUSER_CANARY=1 (debug): a guard region after every symmetric sub-buffer, verified by check_canaries()
        self.guard = 1024 if env_flag("CANARY", 0) else 0
        total = sum(_round_up(v, 1024) + self.guard for v in sizes.values()) + 1024
        self.buf = SymmBuffer(total, group if world > 1 else None, device, guard=self.guard)
        self.off = {k: self.buf.carve(v) for k, v in sizes.items()}
        v = self.buf.view
        self.grecv = v(self.off["grecv"], (max_rows, d_model), dtype)
        self.gcomb = v(self.off["gcomb"], (max_slots, d_model), dtype)
        self.row_src = v(self.off["row_src"], (max_rows,), torch.int32)
        self.row_gate = v(self.off["row_gate"], (max_rows,), torch.float32)
        self.tile_flags = v(self.off["tile_flags"], (max_rows // TILE + 1,), torch.int32)
        self.cnt_table = v(self.off["cnt_table"], (world, e_total), torch.int32)
        self.cnt_flag = v(self.off["cnt_flag"], (N.MAX_RANKS,), torch.int32)
        self.done = v(self.off["done"], (N.MAX_RANKS,), torch.int32)
        self.done_cum = torch.zeros(N.MAX_RANKS, dtype=torch.int32, device=device)
        self.bar_epoch = 0
        self.epoch = 0
        # The epoch can also live on the device (advanced by the plan kernel itself): needed when calls are replayed
        # from a CUDA graph, whose launch arguments are frozen. Switched on by GraphedForward or CCFUSER_DEVICE_EPOCH=1;
        # every rank of the group must switch at the same call.
        self.epoch_dev = torch.zeros(1, dtype=torch.int32, device=device)
        self.device_epoch = bool(env_flag("DEVICE_EPOCH", 0))
        self.ws = G.Workspace.get(device)
        self.users = 0          # fused layers currently attached (FusedMoE.__init__ / close)
        # scratch of the routing kernels
        s_max = max_slots
        nb = (s_max + 1023) // 1024
        self.block_hist = torch.zeros(nb * e_total, dtype=torch.int32, device=device)
        self.block_off = torch.zeros(nb * e_total, dtype=torch.int32, device=device)
        self.ticket = torch.zeros(1, dtype=torch.int32, device=device)
        self.wait_ns = int(float(os.environ.get("CCFUSER_WAIT_LIMIT_S", "5")) * 1e9)
        # CTAs whose epilogue warps run the dispatch role before their first accumulator is due (default: all)
        self.n_comm = env_flag("COMM_CTAS", 1 << 20)

    @classmethod
    def get(cls, group, world, rank, device, max_rows, max_slots, d_model, e_total, dtype) -> "CommContext":
        # keyed on the group's member ranks, not on the group object: object ids are reused after garbage collection
        import torch.distributed as dist
        members = tuple(dist.get_process_group_ranks(group)) if (group is not None and world > 1) else ()
        key = (members, world, str(device), d_model, e_total, dtype)
        ctx = cls._instances.get(key)
        if ctx is None or ctx.max_rows < max_rows or ctx.max_slots < max_slots:
            # (re)allocation is collective: every rank constructs its layers in the same order. A superseded context
            # that no layer uses any more is freed here; one that still has users is freed when its last layer closes.
            if ctx is not None and ctx.users == 0:
                ctx.close()
            ctx = cls(group, world, rank, device, max_rows, max_slots, d_model, e_total, dtype)
            cls._instances[key] = ctx
        return ctx

    def peer(self, name: str):
        return self.buf.peer_ptrs(self.off[name])

    def close(self):
        """Free this context's symmetric buffers (collective over its group; call after the layers that use it have
        been released and their work has completed)."""
        if self.buf is None:
            return
        for name in ("grecv", "gcomb", "row_src", "row_gate", "tile_flags", "cnt_table", "cnt_flag", "done"):
            setattr(self, name, None)
        self.buf.close()
        self.buf = None
        for k, v in list(self._instances.items()):
            if v is self:
                del self._instances[k]

    @classmethod
    def close_all(cls):
        """Free every communication context of this process (collective; e.g. before destroying the process group)."""
        for ctx in list(cls._instances.values()):
            ctx.close()

    def device_barrier(self):
        """On-stream barrier over the ranks of this context's group (collective): returns at once on the host; work
        queued on the stream after it starts only when every rank's stream has reached its barrier. Bounded like every
        device wait: a missing rank ends it with a time-out status instead of a hang."""
        self.bar_epoch += 1
        a = N.BarrierArgs()
        for r, p in enumerate(self.peer("bar_flag")):
            a.peer_flag[r] = p
        a.status, a.wait_limit_ns = self.ws.status.data_ptr(), self.wait_ns
        a.world, a.my_rank, a.epoch = self.world, self.rank, self.bar_epoch
        N.check(N.load().ccf_flag_barrier(C.byref(a), N.stream_ptr()), "ccf_flag_barrier")
        N.count(1)

    def check_canaries(self, extra=()):
        """Debug (CCFUSER_CANARY=1): raise MoECommError if a write ran past the end of a symmetric sub-buffer of this
        context or of the buffers in ``extra``. Reads device memory, so it synchronises."""
        from ..errors import MoECommError
        for buf in (self.buf,) + tuple(extra):
            bad = buf.check_guards()
            if bad:
                raise MoECommError(f"guard region overwritten at byte offsets {bad} of a symmetric buffer "
                                   f"(rank {self.rank}): a kernel wrote past the end of a sub-buffer")

    def use_device_epoch(self):
        """Move the call epoch into device memory (collective in effect: all ranks of the group at the same call)."""
        if not self.device_epoch:
            self.epoch_dev.fill_(self.epoch)
            self.device_epoch = True

    def check_status(self, what="fused MoE"):
        self.ws.check(what)


class _TopKSoftmax(torch.autograd.Function):
    """idx, w = top-k + softmax over the selected logits (csrc/moe_kernels.cu)."""

    @staticmethod
    def forward(ctx, logits, k):
        lib = N.load()
        t, e = logits.shape
        logits = logits.contiguous()
        idx = torch.empty(t, k, dtype=torch.int32, device=logits.device)
        w = torch.empty(t, k, dtype=torch.float32, device=logits.device)
        N.check(lib.ccf_topk_softmax(logits.data_ptr(), int(logits.dtype == torch.float16),
                                     int(logits.dtype == torch.float32), t, e, k, idx.data_ptr(), w.data_ptr(),
                                     N.stream_ptr()), "ccf_topk_softmax")
        N.count(1)
        ctx.save_for_backward(idx, w)
        ctx.e, ctx.dtype = e, logits.dtype
        ctx.mark_non_differentiable(idx)
        return idx, w

    @staticmethod
    def backward(ctx, _gidx, gw):
        lib = N.load()
        idx, w = ctx.saved_tensors
        t, k = idx.shape
        dlogits = torch.zeros(t, ctx.e, dtype=ctx.dtype, device=idx.device)
        gw = gw.contiguous().float()
        N.check(lib.ccf_topk_softmax_bwd(idx.data_ptr(), w.data_ptr(), gw.data_ptr(), t, ctx.e, k,
                                         dlogits.data_ptr(), int(ctx.dtype == torch.float16),
                                         int(ctx.dtype == torch.float32), N.stream_ptr()), "ccf_topk_softmax_bwd")
        N.count(1)
        return dlogits, None


def topk_softmax(logits: torch.Tensor, k: int):
    return _TopKSoftmax.apply(logits, k)


class FusedMoE:
    """Per-layer state of the fused path: symmetric forward buffers, saved activations, launch helpers."""

    def __init__(self, layer):
        cfg = layer.config
        if cfg.dtype not in (torch.bfloat16, torch.float16):
            raise TypeError("the fused backend computes in bf16 or fp16")
        if cfg.d_model % 64 or cfg.d_ffn % 128:
            raise ValueError("fused backend: d_model must be a multiple of 64 and d_ffn a multiple of 128")
        if cfg.num_experts > N.MAX_GROUPS or cfg.ep_size > N.MAX_RANKS or cfg.top_k > 8:
            raise ValueError("fused backend: at most 256 experts, 8 ranks, top-8")
        self.layer, self.cfg = layer, cfg
        self.device = layer.experts.htoh4.weight.device
        self.world, self.rank = cfg.ep_size, layer.ep_rank
        self.max_rows = cfg.max_recv_rows()
        self.max_slots = cfg.max_tokens * cfg.top_k
        if self.max_slots >= (1 << 24):
            raise ValueError("fused backend: max_tokens * top_k must stay below 2^24 (slot ids travel in 24 bits)")
        group = layer.ep_group if self.world > 1 else None
        self.ctx = CommContext.get(group, self.world, self.rank, self.device, self.max_rows, self.max_slots,
                                   cfg.d_model, cfg.num_experts, cfg.dtype)
        self.ctx.users += 1
        # rows of the context may exceed this layer's bound (shared with bigger layers)
        self.max_rows = self.ctx.max_rows
        self.max_slots = self.ctx.max_slots
        nbytes = (_round_up(self.max_rows * cfg.d_model * 2, 1024) + _round_up(self.max_slots * cfg.d_model * 2, 1024)
                  + 2 * self.ctx.guard)
        self.buf = SymmBuffer(nbytes, group, self.device, guard=self.ctx.guard)
        self.off_xrecv = self.buf.carve(self.max_rows * cfg.d_model * 2)
        self.off_comb = self.buf.carve(self.max_slots * cfg.d_model * 2)
        self.xrecv = self.buf.view(self.off_xrecv, (self.max_rows, cfg.d_model), cfg.dtype)
        self.comb = self.buf.view(self.off_comb, (self.max_slots, cfg.d_model), cfg.dtype)
        f = cfg.d_ffn
        dev, dt = self.device, cfg.dtype
        self.h_act = torch.zeros(self.max_rows, f, dtype=dt, device=dev)
        self.h_pre = torch.zeros(self.max_rows, f, dtype=dt, device=dev)
        self.h_pre2 = torch.zeros(self.max_rows, f, dtype=dt, device=dev) if cfg.activation == "swiglu" else None
        e_loc = cfg.experts_per_rank
        i32 = dict(dtype=torch.int32, device=dev)
        self.slot_pos = torch.zeros(self.max_slots, **i32)
        self.slot_row = torch.full((self.max_slots,), -1, **i32)
        self.sorted_slot = torch.zeros(self.max_slots, **i32)        # slot ids in destination order
        self.order_off = torch.zeros(cfg.num_experts + 1, **i32)     # start of each expert in that order; [-1] = kept rows
        self.local_begin = torch.zeros(e_loc, **i32)                 # this rank's own rows inside each local expert
        self.local_rows = torch.zeros(e_loc, **i32)
        self.count_raw = torch.zeros(cfg.num_experts, **i32)
        self.count_kept = torch.zeros(cfg.num_experts, **i32)
        self.dst_base = torch.zeros(cfg.num_experts, **i32)
        self.group_base = torch.zeros(e_loc, **i32)
        self.group_rows = torch.zeros(e_loc, **i32)
        self.sent_rows = torch.zeros(N.MAX_RANKS, **i32)
        self.table_copy = torch.zeros(self.world, cfg.num_experts, **i32)
        self.check_every_call = bool(env_flag("CHECK_STATUS", 0))
        self.fused_router = bool(env_flag("FUSED_ROUTER", 1))   # one-kernel router (ops/router.py) wherever it applies
        self._save_pre = True   # whether the next forward stores the pre-activations (set per call by run_experts)
        # one C call per forward / backward (csrc/runtime.cu); CCFUSER_NATIVE_RUNTIME=0: one Python call per launch
        self.native_runtime = bool(env_flag("NATIVE_RUNTIME", 1))
        self._desc = None
        self._desc_key = None
        self.sgd = None         # (lr, weight decay): expert weights are updated by the weight-gradient GEMMs (fuse_sgd)
        self._call_bn = 256
        self._call_two_cta = None   # kernel choice of the current call's row-grouped launches (_row_two_cta)
        self._owed = None       # weak reference to the autograd node whose backward still needs this layer's buffers

    # ------------------------------------------------------------------------------------------
    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        x = x.contiguous()
        idx, w = self.route(x)
        return self.run_experts(x, idx, w)

    def route(self, x: torch.Tensor):
        """Router logits -> (idx [T, k] int32, weights [T, k] fp32) with the top-k softmax kernel; also sets the gate's
        auxiliary loss."""
        cfg, layer = self.cfg, self.layer
        if x.shape[0] > cfg.max_tokens:
            raise ValueError(f"{x.shape[0]} tokens exceed config.max_tokens={cfg.max_tokens}")
        coef = getattr(layer.gate, "aux_loss_coef", 0.0)
        zcoef = getattr(layer.gate, "z_loss_coef", 0.0)
        lin = getattr(layer.gate, "gate", None)
        if self.fused_router and isinstance(lin, torch.nn.Linear) and R.supported(x, lin.weight, cfg.top_k):
            # linear layer + top-k + softmax in one kernel. The logits are written (fp32) only when an auxiliary loss
            # needs them; their gradient then returns through the same autograd node.
            want = bool((coef and coef > 0) or (zcoef and zcoef > 0))
            if want:
                idx, w, logits = R.fused_router(x, lin.weight, lin.bias, cfg.top_k, want_logits=True)
                loss = router_aux_loss(logits, idx, cfg.num_experts, coef, zcoef)
            else:
                idx, w = R.fused_router(x, lin.weight, lin.bias, cfg.top_k)
                loss = None
            if hasattr(layer.gate, "set_loss"):
                layer.gate.set_loss(loss)
            return idx, w
        logits = layer.gate.logits(x) if hasattr(layer.gate, "logits") else None
        if logits is None:
            raise TypeError("the fused backend needs a gate with a .logits(x) method (NaiveGate)")
        idx, w = topk_softmax(logits, cfg.top_k)
        if hasattr(layer.gate, "set_loss"):
            # auxiliary losses (load balance, z-loss) with the same definition as NaiveGate.forward, kept in torch: a
            # [T, E] reduction next to GEMMs that dominate the layer
            layer.gate.set_loss(router_aux_loss(logits, idx, cfg.num_experts, coef, zcoef))
        return idx, w

    def run_experts(self, x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """The expert-parallel part for given routing decisions. A slot whose expert id is negative is not routed
        (the routing kernels drop it, its gate weight gets a zero gradient from here)."""
        cfg, layer = self.cfg, self.layer
        x = x.contiguous()
        ex = layer.experts
        wg = ex.htoh4_gate.weight if cfg.activation == "swiglu" else None
        bg = ex.htoh4_gate.bias if cfg.activation == "swiglu" else None
        tensors = (x, w, ex.htoh4.weight, ex.htoh4.bias, wg, bg, ex.h4toh.weight, ex.h4toh.bias)
        # without a backward pass to come the pre-activations need not be stored (inference / no_grad)
        self._save_pre = torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors)
        try:
            y = _FusedMoEFn.apply(x, w, idx, ex.htoh4.weight, ex.htoh4.bias, wg, bg, ex.h4toh.weight, ex.h4toh.bias, self)
        finally:
            self._save_pre = True
        if self.check_every_call:
            self.ctx.check_status("fused MoE forward")
        return y

    def native_desc(self) -> N.Layer:
        """The layer's description for the native runtime (csrc/runtime.h: CcfLayer). Built once; rebuilt if a parameter
        tensor has been replaced (its address changed)."""
        cfg, cc, ex = self.cfg, self.ctx, self.layer.experts
        swiglu = cfg.activation == "swiglu"
        params = (ex.htoh4.weight, ex.htoh4.bias, ex.htoh4_gate.weight if swiglu else None,
                  ex.htoh4_gate.bias if swiglu else None, ex.h4toh.weight, ex.h4toh.bias)
        key = tuple(N.ptr(t) for t in params)
        if self._desc is not None and self._desc_key == key:
            return self._desc
        L = N.Layer()
        L.w1, L.b1, L.wg, L.bg, L.w2, L.b2 = key
        L.xrecv, L.comb = self.xrecv.data_ptr(), self.comb.data_ptr()
        L.h_act, L.h_pre, L.h_pre2 = self.h_act.data_ptr(), self.h_pre.data_ptr(), N.ptr(self.h_pre2)
        for name in ("slot_pos", "slot_row", "sorted_slot", "order_off", "local_begin", "local_rows", "count_raw",
                     "count_kept", "dst_base", "group_base", "group_rows", "sent_rows", "table_copy"):
            setattr(L, name, getattr(self, name).data_ptr())
        for name in ("grecv", "gcomb", "row_src", "row_gate", "tile_flags", "done", "done_cum", "block_hist", "block_off",
                     "ticket", "epoch_dev"):
            setattr(L, name, getattr(cc, name).data_ptr())
        L.sched, L.status = cc.ws.sched.data_ptr(), cc.ws.status.data_ptr()
        peers = {"peer_xrecv": self.buf.peer_ptrs(self.off_xrecv), "peer_comb": self.buf.peer_ptrs(self.off_comb),
                 "peer_grecv": cc.peer("grecv"), "peer_gcomb": cc.peer("gcomb"), "peer_row_src": cc.peer("row_src"),
                 "peer_row_gate": cc.peer("row_gate"), "peer_tile_flags": cc.peer("tile_flags"),
                 "peer_cnt_table": cc.peer("cnt_table"), "peer_cnt_flag": cc.peer("cnt_flag"),
                 "peer_done": [p + 4 * self.rank for p in cc.peer("done")]}
        for name, ptrs in peers.items():
            arr = getattr(L, name)
            for r in range(self.world):
                arr[r] = ptrs[r]
        L.wait_limit_ns = cc.wait_ns
        L.d_model, L.d_ffn, L.e_total, L.e_loc, L.top_k = cfg.d_model, cfg.d_ffn, cfg.num_experts, cfg.experts_per_rank, cfg.top_k
        L.world, L.rank = self.world, self.rank
        L.act, L.swiglu, L.fp16 = N.ACT_CODE[cfg.activation], int(swiglu), int(cfg.dtype == torch.float16)
        L.max_rows, L.max_slots = self.max_rows, self.max_slots
        L.n_comm_ctas = min(int(cc.n_comm), 1 << 30)
        L.two_cta = int(G.TWO_CTA_DEFAULT)
        L.comm_warps = int(G.COMM_WARPS_DEFAULT)
        L.small_rows = int(G.SMALL_ROWS_DEFAULT)
        L.device = self.device.index if (self.device.type == "cuda" and self.device.index is not None) else (
            torch.cuda.current_device() if self.device.type == "cuda" else -1)
        self._desc, self._desc_key = L, key
        return L

    # ---- one outstanding forward per layer ----------------------------------------------------------
    def claim_buffers(self, fn_ctx):
        """The saved activations of a forward pass (received rows, pre-activations, activations, routing arrays) live
        in this layer's buffers until its backward pass has run. A second forward in between (an evaluation inside a
        training step, activation checkpointing's recomputation, two micro-batches before one backward) would
        overwrite them and the first backward would silently use the wrong data: raise instead. The claim ends when the
        backward runs or when the autograd graph that holds it is freed."""
        import weakref
        owner = self._owed() if self._owed is not None else None
        if owner is not None and not getattr(owner, "ccf_backward_done", False):
            raise RuntimeError(
                "ccfuser_b200: this MoE layer was called again while the activations saved by its previous forward pass "
                "are still needed by a backward pass that has not run. The fused backend keeps one set of saved "
                "activations per layer: run backward first, call the second forward under torch.no_grad() after it, or "
                "drop the first result (del loss) if no backward will follow.")
        self._owed = weakref.ref(fn_ctx) if self._save_pre else None

    def release_buffers(self, fn_ctx):
        fn_ctx.ccf_backward_done = True
        if self._owed is not None and self._owed() is fn_ctx:
            self._owed = None

    def close(self):
        """Free this layer's symmetric buffers (collective: call on every rank, in the same order of layers). The
        group's shared context goes with its last layer."""
        if self.buf is None:
            return
        self.xrecv = self.comb = None
        self.buf.close()
        self.buf = None
        self.ctx.users -= 1
        if self.ctx.users <= 0:
            self.ctx.close()

    def routing_stats(self):
        """Device tensors describing the last forward call (no host synchronisation): slots per expert before and
        after the capacity clamp on this rank, the [rank, expert] table of kept rows of every rank, rows this rank
        received per local expert."""
        return {"raw_count": self.count_raw, "kept_count": self.count_kept, "count_table": self.table_copy,
                "recv_rows": self.group_rows, "sent_rows": self.sent_rows[:self.world]}

    # ---- launch helpers ------------------------------------------------------------------------
    def _dispatch_args(self, src: torch.Tensor, tokens: int, idx: torch.Tensor, gate_w: torch.Tensor,
                       backward: bool, dgate=None) -> N.DispatchArgs:
        cfg, ctx = self.cfg, self.ctx
        a = N.DispatchArgs()
        a.x = src.data_ptr()
        a.slot_expert = idx.data_ptr()
        a.slot_pos = self.slot_pos.data_ptr()
        a.dst_base = self.dst_base.data_ptr()
        a.slot_gate = gate_w.data_ptr()
        a.saved_comb = self.comb.data_ptr() if backward else 0
        a.dgate = N.ptr(dgate)
        a.slot_row = self.slot_row.data_ptr()
        a.sorted_slot = self.sorted_slot.data_ptr()
        a.order_off = self.order_off.data_ptr()
        a.e_total = cfg.num_experts
        recv = ctx.peer("grecv") if backward else self.buf.peer_ptrs(self.off_xrecv)
        rs, rg, tf = ctx.peer("row_src"), ctx.peer("row_gate"), ctx.peer("tile_flags")
        for r in range(self.world):
            a.peer_recv[r], a.peer_row_src[r], a.peer_row_gate[r], a.peer_tile_flags[r] = recv[r], rs[r], rg[r], tf[r]
        a.work_counter = ctx.ws.sched.data_ptr() + 4 * G.Workspace.DISPATCH_WORK
        a.tokens, a.top_k, a.d = tokens, cfg.top_k, cfg.d_model
        a.capacity = cfg.capacity(tokens)
        a.experts_per_rank, a.my_rank = cfg.experts_per_rank, self.rank
        a.backward, a.fp16, a.max_rows = int(backward), int(cfg.dtype == torch.float16), self.max_rows
        a.total_index = self.max_rows // TILE  # last element of tile_flags: all rows arrived on that rank
        return a

    def _row_two_cta(self, tokens: int):
        """Kernel choice of the row-grouped launches of a call with ``tokens`` tokens per rank: None (the default, CTA
        pairs) or False (one-CTA kernel, 128-row tiles) when an expert expects at most ``CCFUSER_SMALL_ROWS`` rows."""
        rows = tokens * self.cfg.top_k * self.world // max(1, self.cfg.num_experts)
        return None if rows > G.SMALL_ROWS_DEFAULT else False

    def _gemm2_bn(self, tokens: int) -> int:
        """Tile width of the forward GEMM-2 + combine launch of a call with ``tokens`` tokens per rank (ops/gemm.py:
        narrow_tiles); the source-side wait counts its completion units with the same width."""
        rows = tokens * self.cfg.top_k * self.world // max(1, self.cfg.num_experts)
        return G.narrow_tiles(rows, self.cfg.experts_per_rank, self.cfg.d_model, self._row_two_cta(tokens) is False)

    def _combine_kw(self, peer_comb, row_gate):
        ctx = self.ctx
        done = [p + 4 * self.rank for p in ctx.peer("done")]
        return dict(row_src=ctx.row_src, row_gate=row_gate, peer_comb=peer_comb, peer_done=done, world=self.world,
                    send_finish=1, max_slots=self.max_slots)

    def _wait_and_reduce(self, comb: torch.Tensor, tokens: int, n_tiles: int, out: torch.Tensor):
        lib, ctx, cfg = N.load(), self.ctx, self.cfg
        st = N.stream_ptr()
        N.check(lib.ccf_combine_wait(ctx.done.data_ptr(), ctx.done_cum.data_ptr(), self.sent_rows.data_ptr(), n_tiles,
                                     self.world, ctx.wait_ns, ctx.ws.status.data_ptr(), st), "ccf_combine_wait")
        N.check(lib.ccf_combine_reduce(comb.data_ptr(), self.slot_row.data_ptr(), out.data_ptr(), tokens, cfg.top_k,
                                       cfg.d_model, int(cfg.dtype == torch.float16), st), "ccf_combine_reduce")
        N.count(2)


    # ---- forward stages (also used one by one by the kernel benchmark) ---------------------------
    def stage_route_plan(self, idx: torch.Tensor, tokens: int):
        """Positions / kept counts of this rank's slots, count exchange with all ranks, row-layout plan."""
        lib, cfg, cc = N.load(), self.cfg, self.ctx
        st = N.stream_ptr()
        e_tot, e_loc = cfg.num_experts, cfg.experts_per_rank
        N.check(lib.ccf_route_ordered(idx.data_ptr(), tokens * cfg.top_k, e_tot, cfg.capacity(tokens),
                                      self.slot_pos.data_ptr(), cc.block_hist.data_ptr(), cc.block_off.data_ptr(),
                                      self.count_raw.data_ptr(), self.count_kept.data_ptr(), cc.ticket.data_ptr(),
                                      self.order_off.data_ptr(), self.sorted_slot.data_ptr(), self.slot_row.data_ptr(),
                                      self.rank * e_loc, st), "ccf_route_ordered")
        if not cc.device_epoch:
            cc.epoch += 1
        p = N.PlanArgs()
        p.count_kept = self.count_kept.data_ptr()
        tb, fl = cc.peer("cnt_table"), cc.peer("cnt_flag")
        for r in range(self.world):
            p.peer_table[r], p.peer_flag[r] = tb[r], fl[r]
        p.dst_base, p.group_base, p.group_rows = self.dst_base.data_ptr(), self.group_base.data_ptr(), self.group_rows.data_ptr()
        p.sent_rows, p.table_copy, p.status = self.sent_rows.data_ptr(), self.table_copy.data_ptr(), cc.ws.status.data_ptr()
        p.local_begin, p.local_rows = self.local_begin.data_ptr(), self.local_rows.data_ptr()
        p.wait_limit_ns = cc.wait_ns
        p.world, p.my_rank, p.e_total, p.e_loc, p.epoch, p.max_rows = self.world, self.rank, e_tot, e_loc, cc.epoch, self.max_rows
        if cc.device_epoch:
            N.check(lib.ccf_plan_dev_epoch(C.byref(p), cc.epoch_dev.data_ptr(), st), "ccf_plan_dev_epoch")
        else:
            N.check(lib.ccf_plan(C.byref(p), st), "ccf_plan")
        N.count(3)  # route (2 kernels) + plan

    def stage_dispatch_gemm1(self, x, idx, gate_w, w1, b1, wg=None, bg=None, trace=None, save_pre=True, act=None):
        """ONE kernel: push this rank's routed rows to their owners and run GEMM-1 (+ bias + activation) on the rows
        this rank owns, tile by tile as they arrive. ``save_pre=False`` (no backward will follow) skips the stores of
        the pre-activations, which only the activation derivative needs. ``act`` overrides the configured activation
        code of a non-gated FFN (the kernel benchmark times the bare dispatch + GEMM + bias)."""
        cfg, cc = self.cfg, self.ctx
        t, d = x.shape
        f, e_loc = cfg.d_ffn, cfg.experts_per_rank
        disp = self._dispatch_args(x, t, idx, gate_w, backward=False)
        common = dict(group_base=self.group_base, group_rows=self.group_rows, num_groups=e_loc, tile_flags=cc.tile_flags,
                      dispatch=disp, n_comm_ctas=cc.n_comm, wait_ns=cc.wait_ns, workspace=cc.ws, trace=trace,
                      total_index=self.max_rows // TILE, local_begin=self.local_begin, local_rows=self.local_rows,
                      two_cta=self._row_two_cta(t))
        self._call_two_cta = common["two_cta"]
        self._call_bn = self._gemm2_bn(t)
        if cfg.activation == "swiglu":
            G.launch(a0=self.xrecv, b0=w1.view(e_loc * f, d), b1=wg.view(e_loc * f, d), a_major=N.MAJ_K, b_major=N.MAJ_K,
                     epi=N.EPI_SWIGLU, n=f, k=d, b_group_rows=f, out0=self.h_act, out1=self.h_pre if save_pre else None,
                     out2=self.h_pre2 if save_pre else None, bias0=b1, bias1=bg, **common)
        else:
            G.launch(a0=self.xrecv, b0=w1.view(e_loc * f, d), a_major=N.MAJ_K, b_major=N.MAJ_K, epi=N.EPI_BIAS_ACT,
                     n=f, k=d, b_group_rows=f, out0=self.h_act, out1=self.h_pre if save_pre else None, bias0=b1,
                     act=N.ACT_CODE[cfg.activation] if act is None else act, **common)
        cc.tile_flags.zero_()

    def stage_gemm2_combine(self, w2, b2, trace=None):
        """GEMM-2 whose epilogue scales by the gate weight and stores every row into its source rank's combine buffer."""
        cfg, cc = self.cfg, self.ctx
        d, f, e_loc = cfg.d_model, cfg.d_ffn, cfg.experts_per_rank
        G.launch(a0=self.h_act, b0=w2.view(e_loc * d, f), a_major=N.MAJ_K, b_major=N.MAJ_K, epi=N.EPI_COMBINE, n=d, k=f,
                 group_base=self.group_base, group_rows=self.group_rows, num_groups=e_loc, b_group_rows=d, bias0=b2,
                 ld_out=d, wait_ns=cc.wait_ns, workspace=cc.ws, trace=trace, two_cta=self._call_two_cta, bn=self._call_bn,
                 **self._combine_kw(self.buf.peer_ptrs(self.off_comb), cc.row_gate))

    def stage_reduce(self, tokens: int, out: torch.Tensor):
        """Wait until every owner has delivered this rank's rows, then sum the k slots of each token."""
        self._wait_and_reduce(self.comb, tokens, G.combine_units(self.cfg.d_model, self._call_bn), out)


class GraphedForward:
    """Inference forward of one fused MoE layer replayed from a CUDA graph: for the latency-bound regime (a few
    hundred tokens per GPU) where ten kernel launches and their host code cost more than the kernels.

        g = GraphedForward(layer, tokens=256)     # every rank of the group, same point of the program
        y = g(x)                                  # x [n <= 256, d_model]; y [n, d_model] is a view of a buffer that the
                                                  # next call overwrites

    The graph holds the router, routing, plan, both fused GEMMs and the reduce of one call with a fixed token count;
    a call with fewer tokens fills the rest with padding that is masked out of the routing (``token_mask``), so one
    graph serves every batch size up to its own. The cross-GPU protocol is unchanged (flags and counters live in
    device memory; the plan's epoch moves there too, see CommContext.use_device_epoch). Replays are collective like
    eager calls. Status words are not checked inside the graph: call ``layer.check_status()`` when convenient."""

    def __init__(self, layer, tokens: int, warmup: int = 3):
        fm = layer._fused_impl()
        cfg = layer.config
        if tokens > cfg.max_tokens:
            raise ValueError(f"{tokens} tokens exceed config.max_tokens={cfg.max_tokens}")
        fm.ctx.use_device_epoch()
        self.layer, self.tokens = layer, tokens
        # random warm-up input: with zeros every token has the same logits (the router bias), all ranks route everything
        # to the same k experts, and the owners' receive buffers overflow during the warm-up calls
        self.x = torch.randn(tokens, cfg.d_model, device=fm.device).to(cfg.dtype)
        self.valid = torch.ones(tokens, dtype=torch.bool, device=fm.device)
        self._rows = torch.arange(tokens, device=fm.device)
        side = torch.cuda.Stream(device=fm.device)
        side.wait_stream(torch.cuda.current_stream(fm.device))
        fm.ctx.ws.ordered_after()                     # the side stream is ordered after everything issued so far
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(max(1, warmup)):           # first-use set-up (attributes, driver entry points) outside capture
                layer(self.x, token_mask=self.valid)
        torch.cuda.current_stream(fm.device).wait_stream(side)
        fm.ctx.ws.ordered_after()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.y = layer(self.x, token_mask=self.valid)
        fm.ctx.ws.ordered_after()                     # capture ran on torch's capture stream; replays follow the caller's

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        x = x.reshape(-1, self.x.shape[1])
        n = x.shape[0]
        if n > self.tokens:
            raise ValueError(f"{n} tokens exceed the {self.tokens} this graph was captured for")
        self.x[:n].copy_(x)
        torch.lt(self._rows, n, out=self.valid)       # rows beyond n are padding: not routed
        self.graph.replay()
        return self.y[:n]


class GraphedForwardPool:
    """One graph per bucket size; a call uses the smallest bucket that holds its tokens (padding masked out)."""

    def __init__(self, layer, buckets=(128, 512, 2048)):
        self.graphs = [GraphedForward(layer, b) for b in sorted(buckets)]

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        n = x.reshape(-1, x.shape[-1]).shape[0]
        for g in self.graphs:
            if n <= g.tokens:
                return g(x)
        raise ValueError(f"{n} tokens exceed the largest bucket ({self.graphs[-1].tokens})")


class _FusedMoEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate_w, idx, w1, b1, wg, bg, w2, b2, fm: FusedMoE):
        cfg = fm.cfg
        t, d = x.shape
        idx = idx.contiguous()
        gate_w = gate_w.contiguous()
        fm.ctx.ws.enter()
        fm.claim_buffers(ctx)
        if fm.native_runtime:
            y = torch.empty(t, d, dtype=x.dtype, device=x.device)
            cc = fm.ctx
            if not cc.device_epoch:
                cc.epoch += 1
            with nvtx_range("moe.forward_native"):
                N.check(N.load().ccf_layer_forward(C.byref(fm.native_desc()), x.data_ptr(), idx.data_ptr(), gate_w.data_ptr(),
                                                   y.data_ptr(), t, cfg.capacity(t), int(fm._save_pre),
                                                   -1 if cc.device_epoch else cc.epoch, N.stream_ptr(), None, 0, None),
                        "ccf_layer_forward")
            N.count(7)   # kernels: route (2), plan, dispatch + GEMM-1, GEMM-2 + combine, wait, reduce
            ctx.fm = fm
            ctx.tokens = t
            ctx.save_for_backward(idx, gate_w, w1, wg, w2)
            ctx.has_bias = (b1 is not None, bg is not None, b2 is not None)
            return y
        with nvtx_range("moe.route_plan"):
            fm.stage_route_plan(idx, t)
        with nvtx_range("moe.dispatch_gemm1"):
            fm.stage_dispatch_gemm1(x, idx, gate_w, w1, b1, wg, bg, save_pre=fm._save_pre)
        with nvtx_range("moe.gemm2_combine"):
            fm.stage_gemm2_combine(w2, b2)
        y = torch.empty(t, d, dtype=x.dtype, device=x.device)
        with nvtx_range("moe.reduce"):
            fm.stage_reduce(t, y)
        ctx.fm = fm
        ctx.tokens = t
        ctx.save_for_backward(idx, gate_w, w1, wg, w2)
        ctx.has_bias = (b1 is not None, bg is not None, b2 is not None)
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = N.load()
        fm: FusedMoE = ctx.fm
        cfg, cc = fm.cfg, fm.ctx
        cc.ws.enter()
        fm.release_buffers(ctx)
        idx, gate_w, w1, wg, w2 = ctx.saved_tensors
        st = N.stream_ptr()
        t, d, f, e_loc = ctx.tokens, cfg.d_model, cfg.d_ffn, cfg.experts_per_rank
        fp16 = int(cfg.dtype == torch.float16)
        dy = dy.contiguous()
        dgate = torch.zeros(t * cfg.top_k, dtype=torch.float32, device=dy.device)  # dropped slots keep 0
        swiglu = cfg.activation == "swiglu"
        # fuse_sgd: the weight-gradient GEMMs update the weights in place (single-rank layers); no weight gradient is
        # returned, and dgrad-1, which still needs the old w1 / wg, moves in front of them
        # (w2 at any group size; w1 / wg only on a single rank, where dgrad-1 may move in front of their update)
        sgd2 = fm.sgd if (fm.sgd is not None and fm.sgd[0] != 0.0) else None
        sgd = sgd2 if fm.world == 1 else None
        if fm.native_runtime:
            has_b1, has_bg, has_b2 = ctx.has_bias
            mk = lambda like: torch.empty_like(like)                       # noqa: E731
            bias = lambda n: torch.empty(e_loc, n, dtype=cfg.dtype, device=dy.device)   # noqa: E731
            g = N.LayerGrads()
            dh = torch.empty(fm.max_rows, f, dtype=cfg.dtype, device=dy.device)
            dh2 = torch.empty_like(dh) if swiglu else None
            dw2 = None if sgd2 is not None else mk(w2)
            dw1, dwg = (None, None) if sgd is not None else (mk(w1), (mk(wg) if swiglu else None))
            db1, db2, dbg = (bias(f) if has_b1 else None), (bias(d) if has_b2 else None), (bias(f) if has_bg else None)
            dx = torch.empty(t, d, dtype=dy.dtype, device=dy.device)
            g.dgate, g.dh, g.dh2 = dgate.data_ptr(), dh.data_ptr(), N.ptr(dh2)
            g.dw1, g.db1, g.dwg, g.dbg, g.dw2, g.db2, g.dx = (N.ptr(v) for v in (dw1, db1, dwg, dbg, dw2, db2, dx))
            if sgd2 is not None:
                g.sgd_lr, g.sgd_wd = float(sgd2[0]), float(sgd2[1])
            N.check(lib.ccf_layer_backward(C.byref(fm.native_desc()), dy.data_ptr(), idx.data_ptr(), gate_w.data_ptr(),
                                           C.byref(g), t, cfg.capacity(t), st, None, 0, None), "ccf_layer_backward")
            # kernels: dy dispatch + dgrad-2, wgrad-2, wgrad-1 (two for SwiGLU), dgrad-1 + combine, wait, reduce, column sums
            N.count(6 + int(swiglu) + int(has_b1) + int(has_b2) + int(has_bg))
            if fm.check_every_call:
                cc.check_status("fused MoE backward")
            return dx, dgate.view(t, cfg.top_k), None, dw1, db1, dwg, dbg, dw2, db2, None
        # 1+2. push g*dy rows (dispatch role) + dgrad-2 with the activation derivative in the epilogue
        disp = fm._dispatch_args(dy, t, idx, gate_w, backward=True, dgate=dgate)
        common = dict(group_base=fm.group_base, group_rows=fm.group_rows, num_groups=e_loc, wait_ns=cc.wait_ns,
                      workspace=cc.ws)
        dh = torch.empty(fm.max_rows, f, dtype=cfg.dtype, device=dy.device)
        dh2 = torch.empty_like(dh) if swiglu else None
        rt = fm._row_two_cta(t)
        if swiglu:
            G.launch(a0=cc.grecv, b0=w2.view(e_loc * d, f), a_major=N.MAJ_K, b_major=N.MAJ_MN, epi=N.EPI_DSWIGLU, n=f, k=d,
                     b_group_rows=d, out0=dh, out1=dh2, aux0=fm.h_pre, aux1=fm.h_pre2, tile_flags=cc.tile_flags,
                     dispatch=disp, n_comm_ctas=cc.n_comm, total_index=fm.max_rows // TILE, local_begin=fm.local_begin,
                     local_rows=fm.local_rows, two_cta=rt, **common)
        else:
            G.launch(a0=cc.grecv, b0=w2.view(e_loc * d, f), a_major=N.MAJ_K, b_major=N.MAJ_MN, epi=N.EPI_DACT, n=f, k=d,
                     b_group_rows=d, out0=dh, aux0=fm.h_pre, act=N.ACT_CODE[cfg.activation], tile_flags=cc.tile_flags,
                     dispatch=disp, n_comm_ctas=cc.n_comm, total_index=fm.max_rows // TILE, local_begin=fm.local_begin,
                     local_rows=fm.local_rows, two_cta=rt, **common)
        cc.tile_flags.zero_()
        # 3. wgrad-2: dW2[e] = (g dy)^T h_act   [d, f]
        # With few rows per expert the reduction is only a handful of k-blocks and the per-tile latency chain decides:
        # there the one-CTA kernel (shorter barrier round trips, dynamic scheduler) is ~25 % faster than CTA pairs.
        wgrad_two_cta = None if (t * cfg.top_k * fm.world) // max(1, cfg.num_experts) > 512 else False
        dw2 = torch.empty_like(w2) if sgd2 is None else None
        G.launch(a0=cc.grecv, b0=fm.h_act, a_major=N.MAJ_MN, b_major=N.MAJ_MN, epi=N.EPI_STORE, n=f, kgroup=True,
                 m_per_group=d, out0=dw2 if sgd2 is None else w2, ld_out=f, two_cta=wgrad_two_cta, sgd=sgd2, **common)
        has_b1, has_bg, has_b2 = ctx.has_bias

        def colsum(src, n):
            out = torch.empty(e_loc, n, dtype=cfg.dtype, device=dy.device)
            N.check(lib.ccf_colsum_grouped(src.data_ptr(), n, n, e_loc, fm.group_base.data_ptr(),
                                           fm.group_rows.data_ptr(), out.data_ptr(), fp16, st), "ccf_colsum_grouped")
            N.count(1)
            return out

        db2 = colsum(cc.grecv, d) if has_b2 else None
        # 5 (defined here, issued below). dgrad-1 + combine: dx rows go back to the ranks the tokens came from
        def dgrad1():
            ck = fm._combine_kw(cc.peer("gcomb"), None)
            if swiglu:
                G.launch(a0=dh, a1=dh2, b0=wg.view(e_loc * f, d), b1=w1.view(e_loc * f, d), a_major=N.MAJ_K,
                         b_major=N.MAJ_MN, epi=N.EPI_COMBINE, n=d, k=f, kseg=2, b_group_rows=f, ld_out=d, two_cta=rt,
                         **common, **ck)
            else:
                G.launch(a0=dh, b0=w1.view(e_loc * f, d), a_major=N.MAJ_K, b_major=N.MAJ_MN, epi=N.EPI_COMBINE, n=d, k=f,
                         b_group_rows=f, ld_out=d, two_cta=rt, **common, **ck)

        if sgd is not None:
            dgrad1()            # reads w1 / wg before the weight-gradient GEMMs below overwrite them
        # 4. wgrad-1: dW1[e] = dh^T x_e   [f, d]
        dw1 = torch.empty_like(w1) if sgd is None else None
        dwg = dbg = None
        wkw = dict(b0=fm.xrecv, a_major=N.MAJ_MN, b_major=N.MAJ_MN, epi=N.EPI_STORE, n=d, kgroup=True, m_per_group=f, ld_out=d,
                   two_cta=wgrad_two_cta, sgd=sgd, **common)
        if swiglu:
            # dh = d(gate pre-activation), dh2 = d(up pre-activation)
            dwg = torch.empty_like(wg) if sgd is None else None
            G.launch(a0=dh, out0=dwg if sgd is None else wg, **wkw)
            G.launch(a0=dh2, out0=dw1 if sgd is None else w1, **wkw)
            db1 = colsum(dh2, f) if has_b1 else None
            dbg = colsum(dh, f) if has_bg else None
        else:
            G.launch(a0=dh, out0=dw1 if sgd is None else w1, **wkw)
            db1 = colsum(dh, f) if has_b1 else None
        if sgd is None:
            dgrad1()
        dx = torch.empty(t, d, dtype=dy.dtype, device=dy.device)
        fm._wait_and_reduce(cc.gcomb, t, G.combine_units(d), dx)
        if fm.check_every_call:
            cc.check_status("fused MoE backward")
        return dx, dgate.view(t, cfg.top_k), None, dw1, db1, dwg, dbg, dw2, db2, None
