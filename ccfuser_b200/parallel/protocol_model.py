"""Exhaustive check of the cross-GPU synchronisation protocol on an abstract model.

The fused kernels replace the reference's global barriers (``nvshmemx_barrier_all_on_stream`` before and after every
fused GEMM, mix_moe/csrc/mix_moe.h:271,336,420,467) with three kinds of counters (count-exchange epochs, per-tile arrival
counters, per-owner completion counters plus a finish token). Whether that is enough to keep one receive buffer and one
set of counters per role safe across consecutive calls is a question about *all* interleavings of the ranks, which
no run on hardware can show. This module states the protocol as a small transition system and explores every reachable
state:

* every rank runs the same program for ``calls`` consecutive passes (a forward or a backward pass has the same shape:
  plan, push rows, consume rows as owner, return rows, finish, wait as source);
* an action is one atomic step of one rank (a counter update with release semantics, or a wait that is enabled only when
  its condition holds); the explorer interleaves the ranks' actions in every possible order (states are hashed, so the
  search is over states, not over schedules);
* invariants are asserted at the actions they concern: a row of call *i* must find the owner's buffer released from call
  *i - 1*; a count table must not be overwritten before its owner has read the previous exchange; the owner's reset of
  its arrival counters must not lose an arrival; a source's wait for call *i* must not be
  satisfied by anything that belongs to call *i + 1*; and no reachable state may be a deadlock.

``check(...)`` returns the number of states explored or raises ``ProtocolViolation`` with a trace. ``variant`` selects
deliberately broken protocols (used by the tests to show that the explorer finds the hazards the real protocol avoids).
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple


class ProtocolViolation(AssertionError):
    """An invariant of the protocol failed in some reachable interleaving (the message carries the state)."""
    pass


# program of one rank for one call, as a list of step names (expanded per peer / chunk below)
def _program(world: int, chunks: int) -> List[Tuple[str, int, int]]:
    prog: List[Tuple[str, int, int]] = [("publish", 0, 0), ("wait_counts", 0, 0)]
    for o in range(world):
        for c in range(chunks):
            prog.append(("push", o, c))          # rows for owner o, chunk c
    prog.append(("wait_rows", 0, 0))             # owner side: all rows of this call have landed (GEMM-1 tiles)
    prog.append(("reset_tiles", 0, 0))           # stream-ordered after the kernel that consumed the rows
    for s in range(world):
        prog.append(("store", s, 0))             # owner side: results / gradients of source s go back (GEMM-2 epilogue)
    prog.append(("finish", 0, 0))                # last CTA of the owner's last kernel: one token to every rank
    prog.append(("wait_done", 0, 0))             # source side: rows and token from every owner
    return prog


def check(world: int = 2, calls: int = 2, chunks: int = 2, rows: Sequence[Sequence[int]] = None, units: int = 2,
          variant: str = "correct", plan_every: int = 2, max_states: int = 2_000_000) -> int:
    """Explore all interleavings. Only every ``plan_every``-th call exchanges counts (a backward pass reuses the plan of
    its forward pass, so it has no count exchange that would separate it from the call before: there the completion
    counters and the finish token are the only ordering between ranks). ``rows[r][o]`` = rows rank r sends to owner o per call (default 1 + (r + o) % 2 per
    chunk-able unit, scaled by ``chunks``). Variants: 'correct'; 'token_before_store' (finish token sent before the
    results); 'no_token' (sources wait for rows only); 'absolute_targets' (targets not cumulative);
    'reset_after_finish' (arrival counters cleared after the finish token instead of before); 'split_token' (a proposed
    refinement, see the code: token in its own counter, checked per owner just before the next push)."""
    if rows is None:
        rows = [[chunks * (1 + (r + o) % 2) for o in range(world)] for r in range(world)]
    prog = _program(world, chunks)
    if variant == "split_token":
        # Proposed refinement: the finish token travels in a counter of its own. A source waits only for its rows before
        # its reduce, and checks an owner's token just before it next pushes rows to that owner; the owner may then keep
        # working on its buffers after it has returned the rows (owner_tail), e.g. a weight-gradient GEMM placed after
        # the input-gradient GEMM.
        prog = [("publish", 0, 0), ("wait_counts", 0, 0)]
        for o in range(world):
            prog.append(("wait_token", o, 0))
            for c in range(chunks):
                prog.append(("push", o, c))
        prog += [("wait_rows", 0, 0), ("reset_tiles", 0, 0)] + [("store", s_, 0) for s_ in range(world)]
        prog += [("owner_tail", 0, 0), ("finish", 0, 0), ("wait_done", 0, 0)]
    if variant == "token_before_store":
        i, j = prog.index(("finish", 0, 0)), prog.index(("store", 0, 0))
        prog.insert(j, prog.pop(i))
    if variant == "reset_after_finish":
        i = prog.index(("reset_tiles", 0, 0))
        step = prog.pop(i)
        prog.insert(prog.index(("finish", 0, 0)) + 1, step)
    n = len(prog)
    total_steps = n * calls
    # the owner's buffers of a call are in use until the last step of its owner-side work (in the kernels: until the last
    # CTA of the last owner-side kernel, whose epilogue still reads row metadata and, in backward, the saved activations)
    release_at = max(i for i, st in enumerate(prog) if st[0] in ("store", "finish", "owner_tail"))
    expected = [sum(rows[s][o] for s in range(world)) for o in range(world)]     # rows owner o receives per call

    # state: per rank program counter (0 .. total_steps) plus the shared words, all derived data kept explicit
    # words: epoch[o][s], tile[o] (arrival counter), done[s][o], cum[s][o], and bookkeeping for the invariants
    def initial():
        return (tuple([0] * world),                                   # pc
                tuple(tuple([0] * world) for _ in range(world)),      # epoch flags: flag[o][s]
                tuple([0] * world),                                   # tile counter of owner o
                tuple(tuple([0] * world) for _ in range(world)),      # done[s][o]
                tuple(tuple([0] * world) for _ in range(world)),      # cum[s][o]
                tuple(tuple([0] * world) for _ in range(world)),      # stored_calls[s][o]: calls whose rows o has returned to s
                tuple([0] * world),                                   # released[o]: calls whose buffers owner o has let go
                tuple(tuple([0] * world) for _ in range(world)),      # fin[s][o]: finish tokens of owner o seen by s (split_token)
                tuple([0] * world))                                   # tables_read[o]: count exchanges whose table o has consumed

    def fmt(state, who, step):
        return f"rank {who} at call {state[0][who] // n} step {step}; pcs {state[0]}"

    seen = set()
    stack = [initial()]
    seen.add(stack[0])
    explored = 0
    while stack:
        state = stack.pop()
        explored += 1
        if explored > max_states:
            raise RuntimeError("state space larger than max_states")
        pc, epoch, tile, done, cum, stored, released, fin, tables_read = state
        if all(p == total_steps for p in pc):
            continue
        progressed = False
        for r in range(world):
            if pc[r] == total_steps:
                continue
            call, (kind, a, b) = pc[r] // n, prog[pc[r] % n]
            e2, t2, d2, c2, s2, rel2 = [list(x) for x in epoch], list(tile), [list(x) for x in done], \
                [list(x) for x in cum], [list(x) for x in stored], list(released)
            f2 = [list(x) for x in fin]
            tr2 = list(tables_read)
            planned = call % plan_every == 0
            if kind == "publish":
                if planned:
                    nth = call // plan_every                  # this is the nth count exchange (0-based)
                    for o in range(world):
                        if tables_read[o] < nth:
                            raise ProtocolViolation("rank %d overwrites the count table of rank %d, which has not read the "
                                                    "previous exchange yet: %s" % (r, o, fmt(state, r, kind)))
                        e2[o][r] = call + 1
            elif kind == "wait_counts":
                if planned and any(epoch[r][s] < call + 1 for s in range(world)):
                    continue
                if planned:
                    tr2[r] = call // plan_every + 1
            elif kind == "push":
                o = a
                if released[o] < call:
                    raise ProtocolViolation("rows of call %d reach owner %d while it still uses the buffers of call %d: %s"
                                            % (call, o, released[o], fmt(state, r, kind)))
                t2[o] += rows[r][o] // chunks
            elif kind == "wait_rows":
                if tile[r] < expected[r]:
                    continue
                if tile[r] > expected[r]:
                    raise ProtocolViolation("owner %d counts %d rows, more than the %d of call %d: %s"
                                            % (r, tile[r], expected[r], call, fmt(state, r, kind)))
            elif kind == "reset_tiles":
                if tile[r] != expected[r]:
                    raise ProtocolViolation("owner %d clears its arrival counter at %d, not %d: an arrival is lost: %s"
                                            % (r, tile[r], expected[r], fmt(state, r, kind)))
                t2[r] = 0
            elif kind == "store":
                s = a
                d2[s][r] += rows[s][r] * units
                s2[s][r] = call + 1
            elif kind == "wait_token":
                if fin[r][a] < call:      # owner a's token of the previous call (nothing to wait for before the first)
                    continue
            elif kind == "owner_tail":
                pass                      # still reading this call's buffers
            elif kind == "finish":
                if variant == "split_token":
                    for s in range(world):
                        f2[s][r] += 1
                elif variant != "no_token":
                    for s in range(world):
                        d2[s][r] += 1
            elif kind == "wait_done":
                token = 0 if variant in ("no_token", "split_token") else 1
                base = [0] * world if variant == "absolute_targets" else list(cum[r])
                targets = [base[o] + rows[r][o] * units + token for o in range(world)]
                if any(done[r][o] < targets[o] for o in range(world)):
                    continue
                for o in range(world):
                    if stored[r][o] < call + 1:
                        raise ProtocolViolation("rank %d passes its wait of call %d before owner %d has returned its rows: %s"
                                                % (r, call, o, fmt(state, r, kind)))
                    c2[r][o] = targets[o] if variant != "absolute_targets" else 0
            if pc[r] % n == release_at:
                rel2[r] = call + 1
            progressed = True
            p2 = list(pc)
            p2[r] += 1
            nxt = (tuple(p2), tuple(tuple(x) for x in e2), tuple(t2), tuple(tuple(x) for x in d2),
                   tuple(tuple(x) for x in c2), tuple(tuple(x) for x in s2), tuple(rel2), tuple(tuple(x) for x in f2), tuple(tr2))
            if nxt not in seen:
                seen.add(nxt)
                stack.append(nxt)
        if not progressed:
            raise ProtocolViolation(f"deadlock: no rank can move; pcs {pc}, tile {tile}, done {done}, cum {cum}")
    return explored
