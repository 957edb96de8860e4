"""Python launchers of the tcgen05 grouped GEMM (csrc/gemm.cu).

All tensors are 2-byte (bf16 or fp16) CUDA tensors except where noted. ``group_base`` / ``group_rows`` are
int32 device tensors: rows of group ``g`` are ``[group_base[g], group_base[g] + group_rows[g])`` and every
base is a multiple of 128.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import native as N


class Workspace:
    """Per-device scratch the kernels share: tile scheduler counters and the status word."""

    _by_device = {}
    # elements of `sched`: next tile of the dynamic scheduler, CTAs that have finished, chunk claim counter of the
    # dispatch role (each returned to zero by the last CTA of the kernel that used it); the rest is spare
    TILE, FINISHED, DISPATCH_WORK = 0, 1, 2

    def __init__(self, device):
        self.sched = torch.zeros(8, dtype=torch.int32, device=device)
        self.status = torch.zeros(2, dtype=torch.int32, device=device)  # [first hard error, overflow count]
        self._last_stream = None

    @classmethod
    def get(cls, device) -> "Workspace":
        device = torch.device(device)
        if device.type != "cuda":
            key = -1   # host-side dry runs
        else:
            key = device.index if device.index is not None else torch.cuda.current_device()
        ws = cls._by_device.get(key)
        if ws is None:
            ws = cls._by_device[key] = Workspace(device)
        return ws

    def enter(self):
        """Called by every launcher with the stream it is about to launch on. The kernels of one device share this
        workspace's scheduler words, so two calls may only follow each other on different streams if the earlier
        stream has drained (or the caller ordered the streams and says so with ``ordered_after``); work still pending
        on another stream means the two could run concurrently and corrupt each other's tile counters: that raises."""
        if self.sched.device.type != "cuda":
            return
        cur = torch.cuda.current_stream(self.sched.device)
        last = self._last_stream
        if last is not None and last != cur and not torch.cuda.is_current_stream_capturing() and not last.query():
            raise RuntimeError(
                "ccfuser_b200: a fused kernel is being launched on a different CUDA stream while earlier fused work is "
                "still pending on another stream of the same device. The kernels of one device share scheduler words: "
                "issue them on one stream, or order the streams (wait_stream / events) and call "
                "Workspace.get(device).ordered_after() before switching.")
        self._last_stream = cur

    def ordered_after(self):
        """The caller has ordered its next stream after all fused work issued so far (event or wait_stream)."""
        self._last_stream = None

    def check(self, what: str = "kernel"):
        """Host read of the status word; raises if a kernel recorded an error, then clears it."""
        both = self.status.tolist()
        v, overflow = int(both[0]), int(both[1])
        if v or overflow:
            self.status.zero_()
        if overflow and not v:
            from ..errors import MoEOverflow
            raise MoEOverflow(f"{what}: {overflow} rows did not fit a receive buffer and were dropped "
                              f"(raise config.recv_factor or set a capacity_factor)")
        if v:
            code, detail = v & 0xff, v >> 8
            from ..errors import MoECommError, MoECommTimeout, MoEOverflow
            msg = f"{what}: {N.ERR_NAMES.get(code, 'error')}: {describe_status(code, detail)} (code {code}, detail {detail:#x})"
            if code in (1, 2):
                raise MoECommTimeout(msg, where=what, tile=detail)
            if code == 4:
                raise MoEOverflow(msg)
            raise MoECommError(msg)


_MBAR_SITES = {1: "tile scheduler slot (producer)", 2: "free pipeline stage (producer)", 3: "tile index (MMA warp)",
               4: "free accumulator (MMA warp)", 5: "operands of a stage (MMA warp)", 6: "tile index (epilogue)",
               7: "finished accumulator (epilogue)", 0x22: "free pipeline stage (producer, CTA-pair kernel)",
               0x24: "free accumulator (MMA warp, CTA-pair kernel)", 0x25: "operands of a stage (MMA warp, CTA-pair kernel)",
               0x27: "finished accumulator (epilogue, CTA-pair kernel)", 0x40: "free pipeline stage (router producer)",
               0x41: "operands of a stage (router MMA warp)", 0x42: "finished accumulator (router epilogue)"}


def describe_status(code: int, detail: int) -> str:
    """What a recorded status word means: which wait gave up and on whom (the kernels encode the site in `detail`)."""
    if code == 1:
        return "a barrier inside one CTA never completed: waiting for " + _MBAR_SITES.get(detail, f"site {detail:#x}")
    if code == 2:
        if detail & 0xF00000 == 0x800000:
            return f"the count exchange never heard from rank {detail & 0xff} (plan kernel)"
        if detail & 0xF00000 == 0x900000:
            return f"the group barrier never heard from rank {detail & 0xff}"
        if detail & 0xF00000 == 0x400000:
            return f"owner rank {detail & 0xff} never returned all rows and its finish token (combine wait)"
        if detail == 0x123:
            return "a probe wait ran out (test)"
        return f"the rows of receive tile {detail} (rows {detail * 128}..{detail * 128 + 127}) never all arrived"
    if code == 3:
        return f"row {detail} carried an out-of-range source rank or slot (access skipped)"
    if code == 4:
        return f"receive buffer of rank {detail} too small for the rows routed to it"
    return f"unknown code {code}, detail {detail:#x}"


DEFAULT_WAIT_NS = 5_000_000_000
# 256x256 tiles on CTA pairs (tcgen05 cta_group::2) by default; CCFUSER_TWO_CTA=0 selects the one-CTA 128x256 kernel
TWO_CTA_DEFAULT = bool(int(__import__('os').environ.get('CCFUSER_TWO_CTA', '1')))
# 1: the two dedicated dispatch warps of every CTA push the rows (next to the MMA and epilogue warps); 0: the epilogue
# warps push them before their first tile
COMM_WARPS_DEFAULT = int(__import__('os').environ.get('CCFUSER_COMM_WARPS', '1'))
# calls that expect at most this many rows per expert run on the one-CTA kernel's 128-row tiles: around one 256-row pair
# tile per expert most second pair tiles would be padding
SMALL_ROWS_DEFAULT = int(__import__('os').environ.get('CCFUSER_SMALL_ROWS', '320'))


def _is_fp16(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return 1
    if t.dtype == torch.bfloat16:
        return 0
    raise TypeError(f"grouped GEMM operands must be bf16 or fp16, got {t.dtype}")


def launch(*, a0, b0, a_major, b_major, epi, n, k=0, group_base, group_rows, num_groups,
           a1=None, b1=None, kgroup=False, m_per_group=0, kseg=1, b_group_rows=0,
           out0=None, out1=None, out2=None, bias0=None, bias1=None, aux0=None, aux1=None, ld_out=None,
           act=N.ACT_NONE, out_fp32=False, tile_flags=None, local_begin=None, local_rows=None, row_src=None, row_gate=None,
           peer_comb=None, peer_done=None, world=1, send_finish=0, max_slots=0,
           dispatch: Optional[N.DispatchArgs] = None, n_comm_ctas=0, total_index=-1, two_cta=None, wait_ns=DEFAULT_WAIT_NS, grid=0, trace=None,
           workspace: Optional[Workspace] = None, comm_warps: Optional[int] = None, sgd=None, bn: int = 0):
    """Fill a CcfGemmLaunch and launch on the current stream. a0/b0 are 2-D contiguous views."""
    lib = N.load()
    ws = workspace or Workspace.get(a0.device)
    ws.enter()
    L = N.GemmLaunch()
    g = L.args
    g.group_base, g.group_rows = N.ptr(group_base), N.ptr(group_rows)
    g.tile_flags = N.ptr(tile_flags)
    g.local_begin, g.local_rows = N.ptr(local_begin), N.ptr(local_rows)
    g.out0, g.out1, g.out2 = N.ptr(out0), N.ptr(out1), N.ptr(out2)
    g.bias0, g.bias1, g.aux0, g.aux1 = N.ptr(bias0), N.ptr(bias1), N.ptr(aux0), N.ptr(aux1)
    g.row_src, g.row_gate = N.ptr(row_src), N.ptr(row_gate)
    if peer_comb is not None:
        for i, v in enumerate(peer_comb):
            g.peer_comb[i] = v
    if peer_done is not None:
        for i, v in enumerate(peer_done):
            g.peer_done[i] = v
    g.sched, g.status = ws.sched.data_ptr(), ws.status.data_ptr()
    if trace is not None:
        # int64 tensor [grid, tiles, 8]: per tile clock64 stamps {0 tile fetched, 1 rows arrived, 2 last load issued,
        # 3 accumulator free, 4 first operands landed, 5 last MMA committed, 6 accumulator full, 7 epilogue done}
        g.trace, g.trace_tiles = trace.data_ptr(), int(trace.shape[1])
    g.wait_limit_ns = int(wait_ns)
    g.ld_out = int(ld_out if ld_out is not None else n)
    g.n, g.k, g.num_groups, g.m_per_group, g.kseg = int(n), int(k), int(num_groups), int(m_per_group), int(kseg)
    g.b_group_rows, g.act, g.fp16, g.out_fp32 = int(b_group_rows), int(act), _is_fp16(a0), int(bool(out_fp32))
    g.world, g.send_finish, g.n_comm_ctas, g.max_slots = int(world), int(send_finish), int(n_comm_ctas), int(max_slots)
    g.total_index = int(total_index)
    g.comm_warps = int(COMM_WARPS_DEFAULT if comm_warps is None else comm_warps)
    g.bn = int(bn)
    if sgd is not None:     # (lr, weight decay): EPI_STORE updates out0 in place instead of storing the product
        g.sgd_lr, g.sgd_wd = float(sgd[0]), float(sgd[1])
    if dispatch is not None:
        g.disp = dispatch
        g.disp.work_counter = ws.sched.data_ptr() + 4 * Workspace.DISPATCH_WORK
    assert a0.dim() == 2 and b0.dim() == 2 and a0.is_contiguous() and b0.is_contiguous()
    L.a0, L.a1, L.b0, L.b1 = N.ptr(a0), N.ptr(a1), N.ptr(b0), N.ptr(b1)
    L.a_rows, L.a_cols = a0.shape
    L.b_rows, L.b_cols = b0.shape
    L.a_major, L.b_major, L.epi, L.kgroup, L.grid = int(a_major), int(b_major), int(epi), int(bool(kgroup)), int(grid)
    if a0.device.type != "cuda":
        L.device = -1
    else:
        L.device = a0.device.index if a0.device.index is not None else torch.cuda.current_device()
    if two_cta is None:
        two_cta = TWO_CTA_DEFAULT
    # the pair kernel needs 256-row output tiles in k-grouped mode
    L.two_cta = int(bool(two_cta) and not (kgroup and m_per_group % 256 != 0))
    N.check(lib.ccf_gemm_launch(C.byref(L), N.stream_ptr()), "ccf_gemm_launch")
    N.count(1)
    return ws


def combine_units(n: int, bn: int = 256) -> int:
    """Completion-counter increments per output row of a COMBINE GEMM with n columns and bn-column tiles: every tile
    is stored by two epilogue warps per row quarter (one per half of its columns), and each of them reports its rows."""
    return 2 * ((n + bn - 1) // bn)


def narrow_tiles(rows_per_expert: int, experts: int, n: int, one_cta: bool) -> int:
    """Tile width of a row-grouped, K-major-B launch on the one-CTA kernel: 128 when 256-column tiles would leave most of
    the 148 SMs without a tile (a handful of experts with a few hundred rows: the latency-bound serving shapes)."""
    if not one_cta:
        return 256
    tiles = experts * max(1, (rows_per_expert + 127) // 128) * ((n + 255) // 256)
    return 128 if tiles < 148 else 256


def single_group(rows: int, device):
    """group_base / group_rows of an ungrouped GEMM with `rows` rows."""
    return (torch.zeros(1, dtype=torch.int32, device=device),
            torch.full((1,), rows, dtype=torch.int32, device=device))


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, out_fp32: bool = False):
    """y = x @ w.T (+ bias) for 2-D x [M,K], w [N,K]; plain (ungrouped) use of the kernel."""
    m, k = x.shape
    n = w.shape[0]
    out = torch.empty(m, n, dtype=torch.float32 if out_fp32 else x.dtype, device=x.device)
    gb, gr = single_group(m, x.device)
    launch(a0=x.contiguous(), b0=w.contiguous(), a_major=N.MAJ_K, b_major=N.MAJ_K, epi=N.EPI_STORE, n=n, k=k,
           group_base=gb, group_rows=gr, num_groups=1, b_group_rows=n, out0=out,
           bias0=None if bias is None else bias.contiguous(), out_fp32=out_fp32)
    return out
