"""Symmetric device memory: every rank of a group allocates a buffer of the same size and maps all the
others' through CUDA IPC, so kernels can store straight into a peer's HBM over NVLink.

Stands in for the NVSHMEM symmetric heap of the reference (``nvshmem_malloc`` in
mix_moe/csrc/mix_moe.h:75-77 and NVSHMEM's ``peer_heap_base`` table); the exchange of handles goes through
the torch process group instead of MPI. With one rank nothing is exported.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from .. import native as N

_TYPESTR = {torch.bfloat16: None, torch.float16: "<f2", torch.float32: "<f4", torch.int32: "<i4",
            torch.uint8: "|u1", torch.int64: "<i8"}


class _DeviceView:
    """Minimal __cuda_array_interface__ carrier so torch can wrap raw device memory without a copy."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}
        self._owner = owner


def host_id() -> str:
    """Identifies the machine (and boot) this process runs on: CUDA IPC handles are only meaningful inside it."""
    import socket
    boot = ""
    try:
        with open("/proc/sys/kernel/random/boot_id") as f:
            boot = f.read().strip()
    except OSError:
        pass
    return f"{socket.gethostname()}/{boot}"


def check_same_host(hosts: Sequence[str]) -> None:
    """The expert-parallel group exchanges rows through peer memory, so all its ranks must share one NVLink /
    NVSwitch domain, i.e. one machine. Across machines use data parallelism over the expert-parallel groups
    (utils/dist.py: make_ep_dp_groups)."""
    if len(set(hosts)) > 1:
        raise RuntimeError(
            "the ranks of an expert-parallel group must run on one machine (peer memory over NVLink), but this group "
            f"spans {len(set(hosts))}: {sorted(set(hosts))}. Keep ep_size within a node and put data parallelism across nodes "
            "(make_ep_dp_groups(ep_size)).")


class SymmBuffer:
    """One symmetric allocation. ``local`` is a uint8 tensor over this rank's memory; ``peer_ptr(r)``
    is the address at which rank r's copy is mapped in this process."""

    GUARD_BYTE = 0xA5

    def __init__(self, nbytes: int, group=None, device=None, guard: int = 0):
        """``guard`` > 0 (debug): every carved range is followed by that many bytes filled with a fixed pattern that
        no kernel may touch; ``check_guards()`` tells whether a write ran past the end of a range."""
        lib = N.load()
        self.guard = int(guard)
        self._guards: List[int] = []
        self.group = group
        self.world = dist.get_world_size(group) if (dist.is_initialized() and group is not None) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.nbytes = (int(nbytes) + 1023) // 1024 * 1024
        self.device = torch.device(device if device is not None else ("cuda", torch.cuda.current_device()))
        self._opened: List[int] = []
        self._cursor = 0
        if self.device.type != "cuda":
            # Host stand-in for dry runs of the launch logic (native.LaunchRecorder): ordinary host memory, and the
            # peers' base addresses are exchanged as plain numbers that nothing dereferences.
            self.local = torch.zeros(self.nbytes, dtype=torch.uint8)
            self.base = self.local.data_ptr()
            self._peer_base = [self.base]
            if self.world > 1:
                bases: List[Optional[int]] = [None] * self.world
                dist.all_gather_object(bases, self.base, group=group)
                self._peer_base = [int(b) for b in bases]
            self._host = True
            return
        self._host = False
        p = C.c_void_p()
        with torch.cuda.device(self.device):
            N.check(lib.ccf_symm_alloc(self.nbytes, C.byref(p)), "ccf_symm_alloc")
        self.base = p.value
        self._peer_base: List[int] = [0] * self.world
        self._peer_base[self.rank] = self.base
        if self.world > 1:
            hb = lib.ccf_symm_handle_bytes()
            buf = C.create_string_buffer(hb)
            N.check(lib.ccf_symm_get_handle(self.base, buf), "ccf_symm_get_handle")
            gathered: List[Optional[tuple]] = [None] * self.world
            dist.all_gather_object(gathered, (host_id(), bytes(buf.raw)), group=group)
            check_same_host([g[0] for g in gathered])
            handles = [g[1] for g in gathered]
            for r, h in enumerate(handles):
                if r == self.rank:
                    continue
                q = C.c_void_p()
                N.check(lib.ccf_symm_open_handle(C.create_string_buffer(h, hb), C.byref(q)), "ccf_symm_open_handle")
                self._peer_base[r] = q.value
                self._opened.append(q.value)
            dist.barrier(group=group)
        self.local = torch.as_tensor(_DeviceView(self.base, self.nbytes, self), device=self.device)

    def peer_ptr(self, rank: int, offset: int = 0) -> int:
        return self._peer_base[rank] + offset

    def peer_ptrs(self, offset: int = 0) -> List[int]:
        return [b + offset for b in self._peer_base]

    def carve(self, nbytes: int, align: int = 1024) -> int:
        """Bump-allocate a sub-range; every rank must carve in the same order. Returns the byte offset."""
        off = (self._cursor + align - 1) // align * align
        if off + nbytes + self.guard > self.nbytes:
            raise MemoryError(f"symmetric buffer exhausted ({off + nbytes + self.guard} > {self.nbytes})")
        self._cursor = off + nbytes
        if self.guard:
            self.local[self._cursor:self._cursor + self.guard].fill_(self.GUARD_BYTE)
            self._guards.append(self._cursor)
            self._cursor += self.guard
        return off

    def check_guards(self) -> List[int]:
        """Byte offsets of guard regions whose pattern has been overwritten (synchronises with the device)."""
        bad = []
        for off in self._guards:
            if not bool((self.local[off:off + self.guard] == self.GUARD_BYTE).all()):
                bad.append(off)
        return bad

    def view(self, offset: int, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self.local[offset:offset + nbytes].view(dtype).view(*shape)

    def close(self):
        """Unmap the peers' allocations and free this rank's own. Collective over the buffer's group: a rank may only
        free memory that no peer still has mapped or still writes to (freeing an exported allocation under an importer is
        undefined), so every rank first drains its own device work, then all meet, unmap, meet again, and only then
        free. The group's host collectives are bounded by the process group's timeout, so a missing rank ends this with
        an error instead of a hang."""
        if self.base is None:
            return
        if self._host:
            self.local = None
            self.base = None
            return
        lib = N.load()
        multi = self.world > 1 and dist.is_initialized()
        if multi:
            with torch.cuda.device(self.device):
                torch.cuda.synchronize()          # my kernels that store into peers' memory have finished
            dist.barrier(group=self.group)        # ... and so have everyone else's stores into mine
        for q in self._opened:
            lib.ccf_symm_close_handle(q)
        self._opened = []
        if multi:
            dist.barrier(group=self.group)        # nobody maps my allocation any more
        self.local = None
        lib.ccf_symm_free(self.base)
        self.base = None

    def __del__(self):
        # freed explicitly with close(); at interpreter exit the driver reclaims the allocation
        pass
