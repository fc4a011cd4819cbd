"""Loader for the in-tree native libraries (ctypes).

``cuda_lib()`` returns the sm_100a kernel library and raises if it is missing on a
machine with a GPU: the CUDA ops must never silently fall back to eager PyTorch
there.  On a CPU-only machine the ops use their pure-torch reference path and the
library is not needed.
"""
from __future__ import annotations

import ctypes
import os
from functools import lru_cache
from pathlib import Path

import torch

_LIB_DIR = Path(__file__).resolve().parent.parent / "_lib"


class NativeLibraryMissing(RuntimeError):
    pass


#: number of native CUDA entry-point calls made by this process (each launches one or two kernels)
native_calls = 0


class _CountingLib:
    """Proxy over the CDLL that counts calls, so benchmarks can report how many native launches a step made."""

    def __init__(self, dll):
        self._dll = dll
        self._cache = {}

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._dll, name)
            if name.startswith("oslo_") and not name.endswith(("_parts", "_chunk", "_bytes")):

                def fn(*args, _raw=raw):
                    global native_calls
                    native_calls += 1
                    return _raw(*args)
            else:
                fn = raw
            self._cache[name] = fn
        return fn


@lru_cache(maxsize=None)
def cuda_lib():
    return _CountingLib(_load_cuda_lib())


@lru_cache(maxsize=None)
def _load_cuda_lib() -> ctypes.CDLL:
    # OSLO_B200_DEBUG_BOUNDS=1: the library built with index checks that record a status code and skip the access
    debug = os.environ.get("OSLO_B200_DEBUG_BOUNDS", "0") == "1"
    path = _LIB_DIR / ("liboslo_b200_cuda_debug.so" if debug else "liboslo_b200_cuda.so")
    if not path.exists():
        if os.environ.get("OSLO_B200_AUTOBUILD", "1") == "1":
            from oslo_b200.csrc.build import build_cuda

            build_cuda(debug_bounds=debug)
        if not path.exists():
            raise NativeLibraryMissing(
                f"{path} not found: run `python -m oslo_b200.csrc.build` (needs nvcc) before using the CUDA ops"
            )
    return ctypes.CDLL(str(path))


@lru_cache(maxsize=None)
def cpu_lib() -> ctypes.CDLL:
    path = _LIB_DIR / "liboslo_b200_cpu.so"
    if not path.exists():
        from oslo_b200.csrc.build import build_cpu

        build_cpu()
    if not path.exists():
        raise NativeLibraryMissing(f"{path} not found and could not be built (needs g++)")
    return ctypes.CDLL(str(path))


def has_cuda_kernels() -> bool:
    """True when tensors on a CUDA device should take the native-kernel path."""
    return torch.cuda.is_available()


def ptr(t) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


@lru_cache(maxsize=None)
def num_sms(device_index: int = -1) -> int:
    if device_index < 0:
        device_index = torch.cuda.current_device()
    return torch.cuda.get_device_properties(device_index).multi_processor_count


_status_words = {}


def status_word(device=None) -> torch.Tensor:
    """Per-device int32 word where kernels record bounded-wait timeouts (0 = ok)."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    key = (device.type, device.index)
    t = _status_words.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[key] = t
    return t


def check_status(device=None) -> None:
    """Raise if any kernel on ``device`` reported a timeout since the last check (synchronises)."""
    code = int(status_word(device).item())
    if code != 0:
        status_word(device).zero_()
        names = {1: "TMA producer wait", 2: "MMA wait", 3: "epilogue wait", 4: "peer flag wait", 5: "bad argument",
                 6: "index out of bounds (debug build; the access was skipped)"}
        raise RuntimeError(f"oslo_b200 kernel reported status {code} ({names.get(code, 'unknown')})")
