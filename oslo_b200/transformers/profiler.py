"""``FlopsProfiler``: per-module FLOPs / parameters / latency of one forward pass.

Instead of monkey-patching ~40 ``torch.nn.functional`` entry points (the reference's DeepSpeed copy,
oslo/transformers/profiler.py:858-951), FLOPs are counted with a ``TorchDispatchMode`` that sees every ATen matmul /
convolution regardless of how it was reached, plus an explicit counter that the native GEMM wrapper reports into.
Module latencies come from forward pre / post hooks; on CUDA they use events so the device is not synchronised
at every module.
"""
from __future__ import annotations

import time
from collections import defaultdict
from typing import Dict, Optional

import torch
import torch.nn as nn
from torch.utils._python_dispatch import TorchDispatchMode

_ACTIVE: Optional["FlopsProfiler"] = None


def report_gemm_flops(m: int, n: int, k: int, batch: int = 1):
    """Called by the native GEMM wrapper (its kernels are invisible to the ATen dispatcher)."""
    if _ACTIVE is not None:
        _ACTIVE._add(2 * m * n * k * batch)


class _Counter(TorchDispatchMode):
    def __init__(self, prof):
        super().__init__()
        self.prof = prof

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        out = func(*args, **(kwargs or {}))
        name = func.__name__ if hasattr(func, "__name__") else str(func)
        try:
            if name in ("mm.default", "mm"):
                a, b = args[0], args[1]
                self.prof._add(2 * a.shape[0] * a.shape[1] * b.shape[1])
            elif name in ("addmm.default", "addmm"):
                a, b = args[1], args[2]
                self.prof._add(2 * a.shape[0] * a.shape[1] * b.shape[1])
            elif name in ("bmm.default", "bmm", "baddbmm.default"):
                a, b = (args[0], args[1]) if "baddbmm" not in name else (args[1], args[2])
                self.prof._add(2 * a.shape[0] * a.shape[1] * a.shape[2] * b.shape[2])
            elif name.startswith("convolution"):
                x, w = args[0], args[1]
                self.prof._add(2 * out.numel() * (w.numel() // w.shape[0]))
        except Exception:
            pass
        return out


class FlopsProfiler:
    def __init__(self, model: nn.Module):
        self.model = model
        self.flops: Dict[str, int] = defaultdict(int)
        self.latency: Dict[str, float] = defaultdict(float)
        self._stack, self._hooks, self._mode = [], [], None
        self._events = []
        self.started = False

    def _add(self, n: int):
        for name in set(self._stack):
            self.flops[name] += int(n)
        if "" not in self._stack:
            self.flops[""] += int(n)

    def start_profile(self):
        global _ACTIVE
        self.flops.clear()
        self.latency.clear()
        names = {m: n for n, m in self.model.named_modules()}

        def pre(mod, inp):
            name = names[mod]
            self._stack.append(name)
            if torch.cuda.is_available() and any(p.is_cuda for p in mod.parameters(recurse=False)):
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                mod.__prof_t0 = ev
            else:
                mod.__prof_t0 = time.perf_counter()

        def post(mod, inp, out):
            name = self._stack.pop()
            t0 = mod.__prof_t0
            if isinstance(t0, float):
                self.latency[name] += time.perf_counter() - t0
            else:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                self._events.append((name, t0, ev))

        for m in self.model.modules():
            self._hooks.append(m.register_forward_pre_hook(pre))
            self._hooks.append(m.register_forward_hook(post))
        self._mode = _Counter(self)
        self._mode.__enter__()
        _ACTIVE = self
        self.started = True

    def stop_profile(self):
        global _ACTIVE
        if not self.started:
            return
        self._mode.__exit__(None, None, None)
        for h in self._hooks:
            h.remove()
        self._hooks = []
        if self._events:
            torch.cuda.synchronize()
            for name, e0, e1 in self._events:
                self.latency[name] += e0.elapsed_time(e1) / 1e3
            self._events = []
        _ACTIVE = None
        self.started = False

    end_profile = stop_profile

    def get_total_flops(self) -> int:
        return self.flops.get("", 0) or max(self.flops.values(), default=0)

    def get_total_params(self) -> int:
        return sum(p.numel() for p in self.model.parameters())

    def get_total_duration(self) -> float:
        return self.latency.get("", 0.0)

    def print_model_profile(self, top: int = 20, output_file: Optional[str] = None) -> str:
        rows = sorted(((n or "<model>", f, self.latency.get(n, 0.0)) for n, f in self.flops.items()), key=lambda r: -r[1])[:top]
        params = {n or "<model>": sum(p.numel() for p in m.parameters()) for n, m in self.model.named_modules()}
        lines = [f"{'module':60s} {'GFLOPs':>12s} {'params':>14s} {'ms':>10s}"]
        for n, f, t in rows:
            lines.append(f"{n[:60]:60s} {f / 1e9:12.3f} {params.get(n, 0):14d} {t * 1e3:10.3f}")
        text = "\n".join(lines)
        if output_file:
            with open(output_file, "w") as fh:
                fh.write(text + "\n")
        else:
            print(text)
        return text


def get_model_profile(model: nn.Module, kwargs: dict):
    """One profiled forward pass: returns ``(flops, params, seconds)``."""
    prof = FlopsProfiler(model)
    prof.start_profile()
    with torch.no_grad():
        model(**kwargs)
    prof.stop_profile()
    return prof.get_total_flops(), prof.get_total_params(), prof.get_total_duration()
