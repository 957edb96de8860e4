"""Tracing switches. NVTX ranges around the stages of the fused layer are enabled with CCFUSER_NVTX=1 (the reference
only has commented-out NVTX calls, mix_moe/mix_moe/layers.py:509-511,549); ``StageTimer`` collects CUDA-event times per
named stage for the benchmark harness (never inside library launchers)."""
from __future__ import annotations

import contextlib
import os
import time
from collections import defaultdict
from typing import Dict, List

import torch

NVTX = bool(int(os.environ.get("CCFUSER_NVTX", "0")))


@contextlib.contextmanager
def nvtx_range(name: str):
    if NVTX and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class StageTimer:
    """with timer.stage('gemm1'): ... ; timer.summary() -> {stage: mean ms} after a synchronize."""

    def __init__(self):
        self.events: Dict[str, List] = defaultdict(list)

    @contextlib.contextmanager
    def stage(self, name: str):
        if not torch.cuda.is_available():
            # host fallback (CPU backend, tests): wall-clock of the enclosed code
            t0 = time.perf_counter()
            yield
            self.events[name].append((time.perf_counter() - t0) * 1e3)
            return
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        with nvtx_range(name):
            yield
        e.record()
        self.events[name].append((s, e))

    def summary(self) -> Dict[str, float]:
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        return {k: sum(x if isinstance(x, float) else x[0].elapsed_time(x[1]) for x in v) / len(v)
                for k, v in self.events.items()}
