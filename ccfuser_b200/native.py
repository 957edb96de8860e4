"""ctypes binding of the in-tree CUDA library (``ccfuser_b200/lib/libccfuser_b200.so``).

The library exposes plain ``extern "C"`` launchers that take raw device pointers and a stream handle;
the structures below mirror ``csrc/gemm_args.h`` field by field. On a machine with a GPU a missing
library is an error, never a silent fallback to a torch implementation.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

import torch

MAX_RANKS = 8
MAX_GROUPS = 256

EPI_STORE, EPI_BIAS_ACT, EPI_SWIGLU, EPI_COMBINE, EPI_DACT, EPI_DSWIGLU = range(6)
ACT_NONE, ACT_GELU, ACT_RELU = range(3)
MAJ_K, MAJ_MN = 0, 1
ACT_CODE = {"gelu": ACT_GELU, "relu": ACT_RELU, "none": ACT_NONE, "swiglu": ACT_NONE}

ERR_NAMES = {1: "pipeline barrier timeout", 2: "peer flag timeout", 3: "bounds check", 4: "receive buffer overflow"}

_vp = C.c_void_p


class DispatchArgs(C.Structure):
    """Mirror of CcfDispatchArgs (csrc/gemm_args.h)."""
    _fields_ = [
        ("x", _vp), ("slot_expert", _vp), ("slot_pos", _vp), ("dst_base", _vp), ("slot_gate", _vp),
        ("saved_comb", _vp), ("dgate", _vp), ("slot_row", _vp), ("sorted_slot", _vp), ("order_off", _vp),
        ("peer_recv", _vp * MAX_RANKS), ("peer_row_src", _vp * MAX_RANKS),
        ("peer_row_gate", _vp * MAX_RANKS), ("peer_tile_flags", _vp * MAX_RANKS),
        ("work_counter", _vp),
        ("tokens", C.c_int), ("top_k", C.c_int), ("d", C.c_int), ("capacity", C.c_int),
        ("experts_per_rank", C.c_int), ("my_rank", C.c_int), ("backward", C.c_int), ("fp16", C.c_int),
        ("max_rows", C.c_int), ("total_index", C.c_int), ("e_total", C.c_int), ("pad0", C.c_int),
    ]


class GemmArgs(C.Structure):
    """Mirror of CcfGemmArgs (csrc/gemm_args.h)."""
    _fields_ = [
        ("group_base", _vp), ("group_rows", _vp), ("tile_flags", _vp), ("local_begin", _vp), ("local_rows", _vp),
        ("out0", _vp), ("out1", _vp), ("out2", _vp), ("bias0", _vp), ("bias1", _vp), ("aux0", _vp), ("aux1", _vp),
        ("row_src", _vp), ("row_gate", _vp),
        ("peer_comb", _vp * MAX_RANKS), ("peer_done", _vp * MAX_RANKS),
        ("sched", _vp), ("status", _vp), ("trace", _vp),
        ("wait_limit_ns", C.c_ulonglong), ("ld_out", C.c_longlong),
        ("n", C.c_int), ("k", C.c_int), ("num_groups", C.c_int), ("m_per_group", C.c_int), ("kseg", C.c_int),
        ("b_group_rows", C.c_int), ("act", C.c_int), ("fp16", C.c_int), ("out_fp32", C.c_int), ("world", C.c_int),
        ("send_finish", C.c_int), ("n_comm_ctas", C.c_int), ("max_slots", C.c_int), ("trace_tiles", C.c_int),
        ("total_index", C.c_int), ("sgd_lr", C.c_float), ("comm_warps", C.c_int), ("sgd_wd", C.c_float), ("bn", C.c_int), ("pad3", C.c_int),
        ("disp", DispatchArgs),
    ]


class GemmLaunch(C.Structure):
    """Mirror of CcfGemmLaunch (csrc/gemm_args.h)."""
    _fields_ = [
        ("args", GemmArgs),
        ("a0", _vp), ("a1", _vp), ("b0", _vp), ("b1", _vp),
        ("a_rows", C.c_longlong), ("a_cols", C.c_longlong), ("b_rows", C.c_longlong), ("b_cols", C.c_longlong),
        ("a_major", C.c_int), ("b_major", C.c_int), ("epi", C.c_int), ("kgroup", C.c_int), ("grid", C.c_int),
        ("device", C.c_int), ("two_cta", C.c_int), ("pad0", C.c_int),
    ]


class PlanArgs(C.Structure):
    """Mirror of CcfPlanArgs (csrc/gemm_args.h)."""
    _fields_ = [
        ("count_kept", _vp), ("peer_table", _vp * MAX_RANKS), ("peer_flag", _vp * MAX_RANKS),
        ("dst_base", _vp), ("group_base", _vp), ("group_rows", _vp), ("sent_rows", _vp), ("table_copy", _vp),
        ("local_begin", _vp), ("local_rows", _vp),
        ("status", _vp), ("wait_limit_ns", C.c_ulonglong),
        ("world", C.c_int), ("my_rank", C.c_int), ("e_total", C.c_int), ("e_loc", C.c_int), ("epoch", C.c_int),
        ("max_rows", C.c_int),
    ]


class BarrierArgs(C.Structure):
    """Mirror of CcfBarrierArgs (csrc/gemm_args.h)."""
    _fields_ = [("peer_flag", _vp * MAX_RANKS), ("status", _vp), ("wait_limit_ns", C.c_ulonglong),
                ("world", C.c_int), ("my_rank", C.c_int), ("epoch", C.c_int), ("pad0", C.c_int)]


SGD_MULTI = 48


class SgdMulti(C.Structure):
    """Mirror of CcfSgdMulti (csrc/gemm_args.h): up to SGD_MULTI parameter tensors updated by one launch."""
    _fields_ = [("p", _vp * SGD_MULTI), ("g", _vp * SGD_MULTI), ("n", C.c_longlong * SGD_MULTI),
                ("first_block", C.c_int * (SGD_MULTI + 1)), ("count", C.c_int), ("lr", C.c_float), ("wd", C.c_float),
                ("fp16", C.c_int)]


class Layer(C.Structure):
    """Mirror of CcfLayer (csrc/runtime.h): addresses and sizes of one fused layer for the native runtime."""
    _fields_ = [
        ("w1", _vp), ("b1", _vp), ("wg", _vp), ("bg", _vp), ("w2", _vp), ("b2", _vp),
        ("xrecv", _vp), ("comb", _vp), ("h_act", _vp), ("h_pre", _vp), ("h_pre2", _vp),
        ("slot_pos", _vp), ("slot_row", _vp), ("sorted_slot", _vp), ("order_off", _vp), ("local_begin", _vp),
        ("local_rows", _vp), ("count_raw", _vp), ("count_kept", _vp), ("dst_base", _vp), ("group_base", _vp),
        ("group_rows", _vp), ("sent_rows", _vp), ("table_copy", _vp),
        ("grecv", _vp), ("gcomb", _vp), ("row_src", _vp), ("row_gate", _vp), ("tile_flags", _vp), ("done", _vp),
        ("done_cum", _vp), ("block_hist", _vp), ("block_off", _vp), ("ticket", _vp), ("sched", _vp), ("status", _vp),
        ("epoch_dev", _vp),
        ("peer_xrecv", _vp * MAX_RANKS), ("peer_comb", _vp * MAX_RANKS), ("peer_grecv", _vp * MAX_RANKS),
        ("peer_gcomb", _vp * MAX_RANKS), ("peer_row_src", _vp * MAX_RANKS), ("peer_row_gate", _vp * MAX_RANKS),
        ("peer_tile_flags", _vp * MAX_RANKS), ("peer_cnt_table", _vp * MAX_RANKS), ("peer_cnt_flag", _vp * MAX_RANKS),
        ("peer_done", _vp * MAX_RANKS),
        ("wait_limit_ns", C.c_ulonglong),
        ("d_model", C.c_int), ("d_ffn", C.c_int), ("e_total", C.c_int), ("e_loc", C.c_int), ("top_k", C.c_int),
        ("world", C.c_int), ("rank", C.c_int), ("act", C.c_int), ("swiglu", C.c_int), ("fp16", C.c_int),
        ("max_rows", C.c_int), ("max_slots", C.c_int), ("n_comm_ctas", C.c_int), ("two_cta", C.c_int),
        ("device", C.c_int), ("pad0", C.c_int), ("comm_warps", C.c_int), ("small_rows", C.c_int),
    ]


class LayerGrads(C.Structure):
    """Mirror of CcfLayerGrads (csrc/runtime.h)."""
    _fields_ = [("dgate", _vp), ("dh", _vp), ("dh2", _vp), ("dw1", _vp), ("db1", _vp), ("dwg", _vp), ("dbg", _vp),
                ("dw2", _vp), ("db2", _vp), ("dx", _vp), ("sgd_lr", C.c_float), ("sgd_wd", C.c_float)]


_lib = None
_lock = threading.Lock()
LAUNCHES = [0]   # kernels of this library launched by this process (bench.py reports the count)


def count(n: int = 1):
    LAUNCHES[0] += n


def lib_path() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libccfuser_b200.so")


def load(build_if_missing: bool = True):
    """Load (building first if the sources are newer and nvcc exists) and return the ctypes library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = lib_path()
        if build_if_missing:
            from . import build as _build
            try:
                if _build.needs_build():
                    # several ranks of one job may arrive here together: one builds, the others wait for the lock
                    import fcntl
                    os.makedirs(os.path.dirname(path), exist_ok=True)
                    with open(path + ".lock", "w") as lock:
                        fcntl.flock(lock, fcntl.LOCK_EX)
                        try:
                            if _build.needs_build():
                                _build.build()
                        finally:
                            fcntl.flock(lock, fcntl.LOCK_UN)
            except Exception:
                if not os.path.exists(path):
                    raise
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: run `python -m ccfuser_b200.build` (needs nvcc, sm_100a)")
        cdll = C.CDLL(path)
        lib = _DeclaredOnly(cdll, _declare(cdll))
        for name, struct in (("gemm_args", GemmArgs), ("dispatch_args", DispatchArgs),
                             ("gemm_launch", GemmLaunch), ("plan_args", PlanArgs), ("layer", Layer),
                             ("layer_grads", LayerGrads), ("barrier_args", BarrierArgs),
                             ("sgd_multi", SgdMulti)):
            want = getattr(lib, "ccf_sizeof_" + name)()
            if want != C.sizeof(struct):
                raise RuntimeError(f"ctypes mirror of {name} is {C.sizeof(struct)} bytes, library has {want}")
        _lib = lib
        return lib


def _declare(lib):
    i, p, ull, ll = C.c_int, _vp, C.c_ulonglong, C.c_longlong
    sig = {
        "ccf_gemm_launch": ([C.POINTER(GemmLaunch), p], i),
        "ccf_gemm_smem_bytes": ([], i),
        "ccf_debug_pair_tile_order": ([p, p, p, p, i, i, i, i, i, p, i], i),
        "ccf_router_topk": ([p, p, p, i, i, i, i, i, p, p, p, p, ull, i, p], i),
        "ccf_router_select_host": ([p, i, i, i, p, p], i),
        "ccf_router_bwd": ([p, p, p, p, p, p, p, p, i, i, i, i, i, p], i),
        "ccf_topk_softmax": ([p, i, i, i, i, i, p, p, p], i),
        "ccf_topk_softmax_bwd": ([p, p, p, i, i, i, p, i, i, p], i),
        "ccf_route": ([p, i, i, i, p, p, p, p, p, p, p], i),
        "ccf_route_ordered": ([p, i, i, i, p, p, p, p, p, p, p, p, p, i, p], i),
        "ccf_layer_forward": ([C.POINTER(Layer), p, p, p, p, i, i, i, i, p, p, i, p], i),
        "ccf_layer_backward": ([C.POINTER(Layer), p, p, p, C.POINTER(LayerGrads), i, i, p, p, i, p], i),
        "ccf_flag_barrier": ([C.POINTER(BarrierArgs), p], i),
        "ccf_plan": ([C.POINTER(PlanArgs), p], i),
        "ccf_plan_dev_epoch": ([C.POINTER(PlanArgs), p, p], i),
        "ccf_dispatch": ([C.POINTER(DispatchArgs), p, p, i, p], i),
        "ccf_combine_wait": ([p, p, p, i, i, ull, p, p], i),
        "ccf_combine_reduce": ([p, p, p, i, i, i, i, p], i),
        "ccf_colsum_grouped": ([p, ll, i, i, p, p, p, i, p], i),
        "ccf_wait_probe": ([p, i, ull, p, p], i),
        "ccf_sgd_step": ([p, p, ll, C.c_float, C.c_float, i, p], i),
        "ccf_sgd_multi": ([C.POINTER(SgdMulti), p], i),
        "ccf_layernorm_max_d": ([], i),
        "ccf_layernorm_fwd": ([p, p, p, p, p, p, i, i, C.c_float, i, p], i),
        "ccf_layernorm_bwd": ([p, p, p, p, p, p, p, p, i, i, i, p], i),
        "ccf_symm_alloc": ([ull, C.POINTER(p)], i),
        "ccf_symm_free": ([p], i),
        "ccf_symm_handle_bytes": ([], i),
        "ccf_symm_get_handle": ([p, p], i),
        "ccf_symm_open_handle": ([p, C.POINTER(p)], i),
        "ccf_symm_close_handle": ([p], i),
        "ccf_error_string": ([i], C.c_char_p),
    }
    for name, (argtypes, restype) in sig.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = restype
    return set(sig)


class _DeclaredOnly:
    """The loaded library, restricted to the entry points whose signatures are declared above. ctypes would call any
    other exported symbol with its default conversion (Python integers become 32-bit C ints), which silently truncates
    device addresses; an undeclared name is therefore an error here, not a call."""

    def __init__(self, cdll, declared):
        self._cdll, self._declared = cdll, declared

    def __getattr__(self, name):
        if name.startswith("ccf_sizeof_") or name in self._declared:
            return getattr(self._cdll, name)
        raise AttributeError(f"{name}: no signature declared in ccfuser_b200/native.py (_declare)")


class LaunchRecorder:
    """Stands in for the library and records every launcher call instead of running it, so the host side of the fused
    path (which launches, in which order, with which argument blocks) can be tested on a machine without a GPU.
    Size queries and error strings go to the real library; everything else returns 0. Structures passed with
    ``ctypes.byref`` are stored as their raw bytes (``GemmLaunch.from_buffer_copy`` turns them back into fields)."""

    _PASS_THROUGH = ("ccf_sizeof_", "ccf_error_string", "ccf_gemm_smem_bytes", "ccf_symm_handle_bytes")

    def __init__(self, real):
        self._real = real
        self.calls = []

    def __getattr__(self, name):
        fn = getattr(self._real, name)
        if name.startswith(self._PASS_THROUGH):
            return fn

        def record(*args):
            self.calls.append((name, tuple(bytes(a._obj) if hasattr(a, "_obj") else a for a in args)))
            return 0
        return record

    def names(self):
        return [c[0] for c in self.calls]


class record_launches:
    """Context manager: ``with record_launches() as rec: ...`` routes all library calls of this process to a
    LaunchRecorder (no kernel runs, outputs stay uninitialised)."""

    def __enter__(self):
        global _lib
        self._saved = load()
        self.rec = LaunchRecorder(self._saved)
        _lib = self.rec
        return self.rec

    def __exit__(self, *exc):
        global _lib
        _lib = self._saved
        return False


# Argument checks of the host launchers return small negative numbers before any CUDA call is made; failures of CUDA
# calls come back as minus the cudaError_t value. The two ranges overlap for -2 ... -9, so a message names both readings.
ARG_ERRORS = {-2: "argument out of range", -3: "n must be a multiple of 32", -4: "k-grouped GEMM needs m_per_group % 128 == 0",
              -5: "k must be a multiple of 8", -6: "no kernel for this combination of operand majors and epilogue",
              -7: "cudaSetDevice failed", -8: "the CTA-pair kernel needs m_per_group % 256 == 0 in k-grouped mode",
              -9: "the dispatch role exists only in the kernels that read the receive buffer (forward: bias+activation / "
                  "SwiGLU epilogues with backward=0, backward: activation-derivative epilogues with backward=1)",
              -10: "128-column tiles exist in the one-CTA kernel for row-grouped launches with a K-major B operand only"}


def check(rc: int, what: str):
    if rc != 0:
        parts = []
        if rc in ARG_ERRORS:
            parts.append("argument check: " + ARG_ERRORS[rc])
        if -1000 < rc < 0:
            try:
                parts.append("or CUDA error %d: %s" % (-rc, load().ccf_error_string(rc).decode()) if parts else
                             "CUDA error %d: %s" % (-rc, load().ccf_error_string(rc).decode()))
            except Exception:
                pass
        elif rc <= -1000:
            parts.append("driver error %d while encoding a tensor map" % (-rc - 1000))
        raise RuntimeError(f"{what} failed with code {rc} ({'; '.join(parts)})")


def stream_ptr() -> int:
    if not torch.cuda.is_available():
        return 0   # host-side dry runs (LaunchRecorder)
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int:
    """Device address of a tensor (0 for None)."""
    return 0 if t is None else t.data_ptr()
