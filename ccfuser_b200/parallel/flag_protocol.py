"""Host emulation of the device-side push / arrival-counter / completion-counter protocol.

The fused kernels synchronise GPUs with three kinds of words that live in the consumer's memory:

* ``tile_flags[tile]``   rows that have landed in a 128-row tile of a receive buffer (reset by the owner after use);
* ``cnt_flag[src]``      epoch of the last count row written by rank ``src`` (monotonic);
* ``done[owner]``        rows (x column units) an owner has stored into this rank's combine buffer plus one token per
                         finished call (monotonic; the waiter keeps the cumulative target).

This module runs the same protocol with Python threads and numpy buffers so that its ordering properties and its
failure behaviour can be tested without a GPU: arrivals in any order, a sender that never sends (the bounded wait
ends with ``MoECommTimeout``), an owner that runs ahead by one call (its early token must not satisfy the current
wait). The reference has no such protocol: it separates phases with ``nvshmemx_barrier_all_on_stream``
(mix_moe/csrc/mix_moe.h:271,420) and hangs if a rank is missing.
"""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional, Sequence

import numpy as np

from ..errors import MoECommTimeout

TILE = 128


class EmulatedRank:
    """The words of one rank that its peers write (receive buffer, arrival counters, combine buffer, completion counters)
    with the operations peers perform on them and the bounded waits of the owner."""
    def __init__(self, rank: int, world: int, max_rows: int, max_slots: int, d: int):
        self.rank, self.world = rank, world
        self.recv = np.zeros((max_rows, d), dtype=np.float32)
        self.row_src = np.full(max_rows, -1, dtype=np.int64)
        self.tile_flags = np.zeros(max_rows // TILE + 1, dtype=np.int64)
        self.comb = np.zeros((max_slots, d), dtype=np.float32)
        self.done = np.zeros(world, dtype=np.int64)
        self.done_cum = np.zeros(world, dtype=np.int64)
        self.cnt_table = np.zeros((world, 0), dtype=np.int64)
        self.cnt_flag = np.zeros(world, dtype=np.int64)
        self.lock = threading.Lock()      # stands in for the atomicity of red.add
        self.cv = threading.Condition(self.lock)

    # ---- words written by peers ---------------------------------------------------------------
    def push_row(self, src_rank: int, slot: int, row: int, data: np.ndarray):
        """What a dispatch warp does: store the row and its metadata, then release-add the tile counter."""
        self.recv[row] = data
        self.row_src[row] = (src_rank << 24) | slot
        with self.cv:
            self.tile_flags[row // TILE] += 1
            self.cv.notify_all()

    def store_combined(self, owner: int, slot: int, data: np.ndarray, units: int = 1):
        self.comb[slot] = data
        with self.cv:
            self.done[owner] += units
            self.cv.notify_all()

    def finish_token(self, owner: int):
        with self.cv:
            self.done[owner] += 1
            self.cv.notify_all()

    # ---- bounded waits --------------------------------------------------------------------------
    def wait_tile(self, tile: int, expected: int, timeout_s: float):
        deadline = time.monotonic() + timeout_s
        with self.cv:
            while self.tile_flags[tile] < expected:
                left = deadline - time.monotonic()
                if left <= 0:
                    raise MoECommTimeout(f"rank {self.rank}: tile {tile} has {int(self.tile_flags[tile])}/{expected} rows",
                                         where="tile_flags", tile=tile)
                self.cv.wait(left)

    def reset_tiles(self):
        with self.cv:
            self.tile_flags[:] = 0

    def wait_combine(self, sent_rows: Sequence[int], units: int, timeout_s: float):
        """Per-owner cumulative targets: rows sent to that owner x units + one finish token."""
        deadline = time.monotonic() + timeout_s
        targets = [int(self.done_cum[o]) + int(sent_rows[o]) * units + 1 for o in range(self.world)]
        with self.cv:
            for o, tgt in enumerate(targets):
                while self.done[o] < tgt:
                    left = deadline - time.monotonic()
                    if left <= 0:
                        raise MoECommTimeout(f"rank {self.rank}: owner {o} delivered {int(self.done[o])} of {tgt}",
                                             where="done", peer=o)
                    self.cv.wait(left)
            self.done_cum[:] = targets


def run_call(ranks: List[EmulatedRank], plans: List[Dict], expert_fn, timeout_s: float = 2.0,
             drop_sender: Optional[int] = None, shuffle_seed: Optional[int] = None, units: int = 2):
    """One forward call on all emulated ranks, each rank in its own thread.

    plans[r] = {'x': [T, d] array, 'slot_owner': [S], 'slot_row': [S] (-1 = dropped), 'top_k': k,
                'tiles': {owner-side: list of (tile, expected_rows)}}.
    ``drop_sender`` makes one rank skip its dispatch (fault injection on the host).
    Returns the per-rank reduced outputs; raises MoECommTimeout from the first rank whose wait ran out.
    """
    world = len(ranks)
    outs: List[Optional[np.ndarray]] = [None] * world
    errors: List[Optional[BaseException]] = [None] * world

    def body(r: int):
        me, plan = ranks[r], plans[r]
        try:
            k = plan["top_k"]
            order = np.arange(len(plan["slot_row"]))
            if shuffle_seed is not None:
                np.random.RandomState(shuffle_seed + r).shuffle(order)
            if drop_sender != r:
                for s in order:
                    row = int(plan["slot_row"][s])
                    if row >= 0:
                        ranks[int(plan["slot_owner"][s])].push_row(r, int(s), row, plan["x"][s // k])
            # owner side: tile by tile as rows land
            for tile, expected in plan["tiles"]:
                me.wait_tile(tile, expected, timeout_s)
                lo = tile * TILE
                for row in range(lo, lo + expected):
                    packed = int(me.row_src[row])
                    src, slot = packed >> 24, packed & 0xffffff
                    y = expert_fn(r, row, me.recv[row])
                    ranks[src].store_combined(r, slot, y, units)
            me.reset_tiles()
            for peer in ranks:
                peer.finish_token(r)
            # source side
            sent = [int(((plan["slot_owner"] == o) & (plan["slot_row"] >= 0)).sum()) for o in range(world)]
            me.wait_combine(sent, units, timeout_s)
            t = len(plan["x"])
            keep = (plan["slot_row"] >= 0).reshape(t, k, 1)
            outs[r] = (me.comb[:t * k].reshape(t, k, -1) * keep).sum(1)
        except BaseException as e:  # noqa: BLE001 - reported to the caller
            errors[r] = e

    threads = [threading.Thread(target=body, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout_s * 4 + 5)
    for e in errors:
        if e is not None:
            raise e
    return outs
