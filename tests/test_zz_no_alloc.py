"""The allocation-free routing entry point, called through its exported C symbol.

It serves host programs that cannot allocate on the device while they run (their own pool owns the whole
GPU, or a cudaMalloc in their loop is not acceptable), so its kernels use a fixed scratch array inside
the library. The test checks that it gives exactly what the regular entry point (`ccf_route`, scratch
supplied by the caller) gives, on two calls in a row: the second call meets the scratch contents the
first one left behind. This file sorts last so that a failure here cannot hide another test's result.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from ccfuser_b200 import native as N
    N.load()
    lib = C.CDLL(N.lib_path())  # the plain exported symbols, as a C caller would see them
    lib.ccf_route_noalloc.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.ccf_route_noalloc.restype = C.c_int
    lib.ccf_route_noalloc_strerror.argtypes = [C.c_int]
    lib.ccf_route_noalloc_strerror.restype = C.c_char_p
    return lib


def _regular(expert, s, e, cap):
    from ccfuser_b200 import native as N
    lib = N.load()
    nb = (s + 1023) // 1024
    dev = expert.device
    pos = torch.empty(s, dtype=torch.int32, device=dev)
    bh = torch.zeros(nb * e, dtype=torch.int32, device=dev)
    bo = torch.zeros(nb * e, dtype=torch.int32, device=dev)
    raw = torch.zeros(e, dtype=torch.int32, device=dev)
    kept = torch.zeros(e, dtype=torch.int32, device=dev)
    ticket = torch.zeros(1, dtype=torch.int32, device=dev)
    N.check(lib.ccf_route(expert.data_ptr(), s, e, cap, pos.data_ptr(), bh.data_ptr(), bo.data_ptr(), raw.data_ptr(),
                          kept.data_ptr(), ticket.data_ptr(), N.stream_ptr()), "ccf_route")
    return pos, raw, kept


def test_no_alloc_route_matches_regular_entry_point_twice():
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: the second one is smaller, so stale scratch from the first is in reach
    for s, e, cap, seed in [(40000, 64, 900, 1), (5000, 200, 17, 2)]:
        g = torch.Generator().manual_seed(seed)
        p = torch.rand(e, generator=g).pow(2)
        expert = torch.multinomial(p / p.sum(), s, replacement=True, generator=g).int()
        expert[::97] = -1  # ids out of range are skipped by both entry points
        expert = expert.cuda()
        pos = torch.full((s,), -7, dtype=torch.int32, device="cuda")
        raw = torch.full((e,), -7, dtype=torch.int32, device="cuda")
        kept = torch.full((e,), -7, dtype=torch.int32, device="cuda")
        rc = lib.ccf_route_noalloc(expert.data_ptr(), s, e, cap, pos.data_ptr(), raw.data_ptr(), kept.data_ptr(), stream)
        assert rc == 0, lib.ccf_route_noalloc_strerror(rc).decode()
        torch.cuda.synchronize()
        rpos, rraw, rkept = _regular(expert, s, e, cap)
        torch.cuda.synchronize()
        assert torch.equal(pos, rpos)
        assert torch.equal(raw, rraw)
        assert torch.equal(kept, rkept)


def test_no_alloc_route_rejects_sizes_beyond_its_scratch():
    lib = _lib()
    x = torch.zeros(8, dtype=torch.int32, device="cuda")
    for s, e in [(65537, 8), (16, 257), (-1, 8), (16, 0)]:
        rc = lib.ccf_route_noalloc(x.data_ptr(), s, e, 4, x.data_ptr(), x.data_ptr(), x.data_ptr(), None)
        assert rc == -2
        assert b"65536" in lib.ccf_route_noalloc_strerror(rc)
    torch.cuda.synchronize()
