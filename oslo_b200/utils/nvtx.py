"""NVTX ranges and per-path CUDA-event timers around the fused paths (tracing aid).

``OSLO_B200_NVTX=1`` (or ``enable()``) makes every ``annotate("name")`` block push / pop an NVTX range, so the fused
collective, ZeRO, MoE, loss and attention launches show up by name on a profiler timeline.  ``timers()`` additionally
accumulates device time per name with CUDA events, read back with ``summary()`` (the events are only resolved there, so
a training step is not synchronised).  Both are off by default and cost one attribute test per call when off.
"""
from __future__ import annotations

import os
from collections import defaultdict
from contextlib import contextmanager

import torch

_nvtx = os.environ.get("OSLO_B200_NVTX", "0") == "1"
_timing = False
_events = defaultdict(list)


def enable(nvtx: bool = True, timers: bool = False):
    global _nvtx, _timing
    _nvtx, _timing = nvtx, timers


def disable():
    enable(False, False)


@contextmanager
def annotate(name: str):
    """``with annotate("ag_gemm"): ...``"""
    if not (_nvtx or _timing) or not torch.cuda.is_available():
        yield
        return
    if _nvtx:
        torch.cuda.nvtx.range_push(name)
    e0 = e1 = None
    if _timing:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    try:
        yield
    finally:
        if _timing:
            e1.record()
            _events[name].append((e0, e1))
        if _nvtx:
            torch.cuda.nvtx.range_pop()


def summary(reset: bool = True) -> dict:
    """``{name: (calls, total_ms)}`` of everything timed since the last reset (synchronises the device)."""
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    out = {name: (len(ev), sum(a.elapsed_time(b) for a, b in ev)) for name, ev in _events.items()}
    if reset:
        _events.clear()
    return out
