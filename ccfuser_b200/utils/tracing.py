"""Tracing switches. NVTX ranges around the stages of the fused layer are enabled with CCFUSER_NVTX=1 (the reference
only has commented-out NVTX calls, mix_moe/mix_moe/layers.py:509-511,549); ``StageTimer`` collects CUDA-event times per
named stage for the benchmark harness (never inside library launchers)."""
from __future__ import annotations

import contextlib
import os
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
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        with nvtx_range(name):
            yield
        e.record()
        self.events[name].append((s, e))

    def summary(self) -> Dict[str, float]:
        torch.cuda.synchronize()
        return {k: sum(a.elapsed_time(b) for a, b in v) / len(v) for k, v in self.events.items()}
