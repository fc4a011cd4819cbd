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


def report_op_flops(flops: int, macs: int = 0):
    """Called by the other native op wrappers (fused attention, norms, ...)."""
    if _ACTIVE is not None:
        _ACTIVE._add(flops, macs)


# ATen operators counted at one FLOP per output element (activations, pointwise arithmetic, pooling, up-sampling), the
# functional entry points of the reference's table (relu ... tanh, softmax, add / mul, pool / upsample:
# oslo/transformers/profiler.py:858-951) all land on one of these whichever Python API was used
_PER_ELEMENT = (
    "relu", "relu_", "leaky_relu", "leaky_relu_", "elu", "elu_", "prelu", "relu6", "hardtanh", "hardtanh_", "silu", "silu_",
    "gelu", "sigmoid", "sigmoid_", "tanh", "tanh_", "hardswish", "hardsigmoid", "softplus", "mish", "threshold", "threshold_",
    "add", "add_", "sub", "sub_", "mul", "mul_", "div", "div_", "rsub", "neg", "exp", "log", "sqrt", "rsqrt", "pow",
    "_softmax", "_log_softmax", "softmax", "log_softmax",
    "avg_pool1d", "avg_pool2d", "avg_pool3d", "max_pool2d_with_indices", "max_pool3d_with_indices", "adaptive_avg_pool2d",
    "_adaptive_avg_pool2d", "adaptive_max_pool2d", "upsample_nearest1d", "upsample_nearest2d", "upsample_nearest3d",
    "upsample_bilinear2d", "upsample_bicubic2d", "upsample_linear1d", "upsample_trilinear3d",
)
# normalisations: mean, variance, normalise, scale, shift
_NORMS = {"native_layer_norm": 5, "native_batch_norm": 5, "_native_batch_norm_legit": 5, "_native_batch_norm_legit_no_training": 5,
          "native_group_norm": 5, "instance_norm": 5, "cudnn_batch_norm": 5}


class _Counter(TorchDispatchMode):
    def __init__(self, prof):
        super().__init__()
        self.prof = prof

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        out = func(*args, **(kwargs or {}))
        full = func.__name__ if hasattr(func, "__name__") else str(func)
        name = full.split(".")[0]
        try:
            if name == "mm":
                a, b = args[0], args[1]
                macs = a.shape[0] * a.shape[1] * b.shape[1]
                self.prof._add(2 * macs, macs)
            elif name == "addmm":
                a, b = args[1], args[2]
                macs = a.shape[0] * a.shape[1] * b.shape[1]
                self.prof._add(2 * macs + out.numel(), macs)
            elif name in ("bmm", "baddbmm"):
                a, b = (args[0], args[1]) if name == "bmm" else (args[1], args[2])
                macs = a.shape[0] * a.shape[1] * a.shape[2] * b.shape[2]
                self.prof._add(2 * macs, macs)
            elif name.startswith("convolution") or name in ("cudnn_convolution", "mkldnn_convolution"):
                w = args[1]
                macs = out.numel() * (w.numel() // w.shape[0])
                self.prof._add(2 * macs, macs)
            elif name.startswith("_scaled_dot_product") or name == "scaled_dot_product_attention":
                q, k, v = args[0], args[1], args[2]
                macs = q.numel() * k.shape[-2] + q.numel() // q.shape[-1] * k.shape[-2] * v.shape[-1]
                self.prof._add(2 * macs, macs)
            elif name in _NORMS:
                first = out[0] if isinstance(out, (tuple, list)) else out
                self.prof._add(_NORMS[name] * first.numel())
            elif name in _PER_ELEMENT:
                first = out[0] if isinstance(out, (tuple, list)) else out
                if torch.is_tensor(first) and first.is_floating_point():
                    self.prof._add(first.numel())
        except Exception:
            pass
        return out


def number_to_string(num: float, units: Optional[str] = None, precision: int = 2, suffix: str = "") -> str:
    for unit, scale in (("T", 1e12), ("G", 1e9), ("M", 1e6), ("K", 1e3)):
        if units == unit or (units is None and abs(num) >= scale):
            return f"{num / scale:.{precision}f} {unit}{suffix}"
    return f"{num:.{precision}f} {suffix}".rstrip()


def flops_to_string(flops, units=None, precision=2):
    return number_to_string(flops, units, precision, "FLOPs")


def macs_to_string(macs, units=None, precision=2):
    return number_to_string(macs, units, precision, "MACs")


def params_to_string(params, units=None, precision=2):
    return number_to_string(params, units, precision).rstrip()


def duration_to_string(seconds, units=None, precision=2):
    if seconds >= 1 or units == "s":
        return f"{seconds:.{precision}f} s"
    if seconds >= 1e-3 or units == "ms":
        return f"{seconds * 1e3:.{precision}f} ms"
    return f"{seconds * 1e6:.{precision}f} us"


class FlopsProfiler:
    def __init__(self, model: nn.Module):
        self.model = model
        self.flops: Dict[str, int] = defaultdict(int)
        self.macs: Dict[str, int] = defaultdict(int)
        self.latency: Dict[str, float] = defaultdict(float)
        self._stack, self._hooks, self._mode = [], [], None
        self._events = []
        self.started = False

    def _add(self, n: int, macs: int = 0):
        for name in set(self._stack) | ({""} if "" not in self._stack else set()):
            self.flops[name] += int(n)
            self.macs[name] += int(macs)

    def start_profile(self):
        global _ACTIVE
        self.flops.clear()
        self.macs.clear()
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

    def get_total_macs(self) -> int:
        return self.macs.get("", 0) or max(self.macs.values(), default=0)

    def get_total_params(self) -> int:
        return sum(p.numel() for p in self.model.parameters())

    def get_total_duration(self) -> float:
        return self.latency.get("", 0.0)

    def print_model_profile(self, profile_step: int = 1, module_depth: int = -1, top_modules: int = 20, detailed: bool = True,
                            output_file: Optional[str] = None, top: Optional[int] = None) -> str:
        """Summary (totals) followed, when ``detailed``, by the ``top_modules`` heaviest modules down to ``module_depth``
        levels of the module tree (-1 = all levels): FLOPs, MACs, parameters, forward latency and achieved FLOP/s."""
        top_modules = top if top is not None else top_modules
        params = {n: sum(p.numel() for p in m.parameters()) for n, m in self.model.named_modules()}
        total_f, total_m, total_t = self.get_total_flops(), self.get_total_macs(), self.get_total_duration()
        lines = [
            f"profile of step {profile_step}",
            f"params: {params_to_string(self.get_total_params())}   fwd FLOPs: {flops_to_string(total_f)}   fwd MACs: "
            f"{macs_to_string(total_m)}   fwd latency: {duration_to_string(total_t)}   "
            f"fwd FLOP/s: {number_to_string(total_f / total_t if total_t > 0 else 0.0, suffix='FLOP/s')}",
        ]
        if detailed:
            rows = [(n, f) for n, f in self.flops.items() if module_depth < 0 or (n.count(".") + 1 if n else 0) <= module_depth]
            rows = sorted(rows, key=lambda r: -r[1])[:top_modules]
            lines.append(f"{'module':60s} {'GFLOPs':>12s} {'GMACs':>12s} {'params':>14s} {'ms':>10s}")
            for n, f in rows:
                lines.append(f"{(n or '<model>')[:60]:60s} {f / 1e9:12.3f} {self.macs.get(n, 0) / 1e9:12.3f} "
                             f"{params.get(n, 0):14d} {self.latency.get(n, 0.0) * 1e3:10.3f}")
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
