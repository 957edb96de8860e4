"""Host-side failure detection for the process group: heartbeats through the rendezvous store and a bounded
wrapper for collectives. The reference exits on any error and hangs the other ranks in a barrier
(mix_moe/csrc/mix_moe.h:17-25, recorded crash in mix_moe/ae/1:14-36); here a missing rank becomes a
``MoECommTimeout`` on the ranks that are still alive, between steps, with no kernel in flight."""
from __future__ import annotations

import threading
import time
from typing import Callable

import torch.distributed as dist

from ..errors import MoECommTimeout


class Heartbeat:
    """Every rank publishes the last step it finished; ``check`` fails if a peer is more than ``lag`` steps behind
    after ``timeout_s``. ``store`` is any torch.distributed Store (TCPStore, FileStore, HashStore for tests)."""

    def __init__(self, store, rank: int, world: int, prefix: str = "ccfuser/hb"):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix

    def beat(self, step: int):
        self.store.set(f"{self.prefix}/{self.rank}", str(step))

    def peer_step(self, r: int) -> int:
        try:
            return int(self.store.get(f"{self.prefix}/{r}").decode())
        except Exception:
            return -1

    def check(self, step: int, timeout_s: float = 5.0, lag: int = 0, poll_s: float = 0.05):
        deadline = time.monotonic() + timeout_s
        while True:
            late = [r for r in range(self.world) if r != self.rank and self.peer_step(r) < step - lag]
            if not late:
                return
            if time.monotonic() > deadline:
                raise MoECommTimeout(f"rank {self.rank}: ranks {late} did not reach step {step} within {timeout_s}s",
                                     where="heartbeat", peer=late[0])
            time.sleep(poll_s)


def run_with_timeout(fn: Callable[[], object], timeout_s: float, what: str = "collective"):
    """Run ``fn`` (typically a torch.distributed call) in a helper thread; raise MoECommTimeout if it does not return
    in time. The stuck call keeps its thread; callers are expected to tear the process group down afterwards."""
    result, error = [], []

    def target():
        try:
            result.append(fn())
        except BaseException as e:  # noqa: BLE001
            error.append(e)

    th = threading.Thread(target=target, daemon=True)
    th.start()
    th.join(timeout_s)
    if th.is_alive():
        raise MoECommTimeout(f"{what} did not finish within {timeout_s}s", where=what)
    if error:
        raise error[0]
    return result[0] if result else None


def monitored_barrier(group=None, timeout_s: float = 10.0):
    """Barrier that names the missing ranks (gloo) or times out (nccl) instead of waiting forever."""
    import datetime
    if not dist.is_initialized():
        return
    if dist.get_backend(group) == "gloo":
        try:
            dist.monitored_barrier(group=group, timeout=datetime.timedelta(seconds=timeout_s))
        except RuntimeError as e:
            raise MoECommTimeout(str(e), where="monitored_barrier") from e
    else:
        run_with_timeout(lambda: dist.barrier(group=group), timeout_s, "barrier")
