"""Exceptions raised by the communication layer."""


class MoECommError(RuntimeError):
    """A fused kernel reported a non-zero status word."""


class MoECommTimeout(MoECommError):
    """A bounded device- or host-side wait ran out before the peer's data or flag arrived.

    The reference has no such path: a missing rank leaves the others inside
    nvshmemx_barrier_all_on_stream forever (mix_moe/csrc/mix_moe.h:271).
    """

    def __init__(self, msg, *, where=None, peer=None, tile=None):
        super().__init__(msg)
        self.where = where
        self.peer = peer
        self.tile = tile


class MoEOverflow(MoECommError):
    """More rows were routed to a rank than its receive buffer was sized for."""
