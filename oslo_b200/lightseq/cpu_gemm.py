"""Host-side GEMMs for CPU inference (``csrc/cpu/cpu_gemm.cpp``): fp32 and uint8 x int8 -> int32 with per-column
compensation, OpenMP + run-time-selected AVX-512 / AVX2 loops.

Counterpart of the x86 inference GEMM wrappers of the reference's LightSeq subset
(oslo/lightseq2/csrc/kernels/x86/gemm.cpp:10-50).  ``quantized_linear`` shows the intended use: activations quantised to
uint8 with a +128 shift, int8 weights, and the shift removed again through the compensation vector.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from oslo_b200.ops import _lib


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def sgemm(a: torch.Tensor, b: torch.Tensor, transpose_a: bool = False, transpose_b: bool = False, alpha: float = 1.0,
          beta: float = 0.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``alpha * op(a) @ op(b) + beta * out`` for contiguous fp32 CPU matrices."""
    assert a.dtype == torch.float32 and b.dtype == torch.float32 and a.device.type == "cpu" and b.device.type == "cpu"
    a, b = a.contiguous(), b.contiguous()
    m, k = (a.shape[1], a.shape[0]) if transpose_a else a.shape
    kb, n = (b.shape[1], b.shape[0]) if transpose_b else b.shape
    if k != kb:
        raise ValueError(f"inner dimensions differ: {k} vs {kb}")
    if out is None:
        out = torch.zeros(m, n, dtype=torch.float32)
    rc = _lib.cpu_lib().oslo_cpu_sgemm(
        ctypes.c_int(int(transpose_a)), ctypes.c_int(int(transpose_b)), ctypes.c_longlong(m), ctypes.c_longlong(n),
        ctypes.c_longlong(k), ctypes.c_float(alpha), _ptr(a), ctypes.c_longlong(a.stride(0)), _ptr(b),
        ctypes.c_longlong(b.stride(0)), ctypes.c_float(beta), _ptr(out), ctypes.c_longlong(out.stride(0)))
    if rc:
        raise RuntimeError(f"oslo_cpu_sgemm failed ({rc})")
    return out


def gemm_u8s8s32(a: torch.Tensor, b: torch.Tensor, transpose_a: bool = False, transpose_b: bool = False, alpha: float = 1.0,
                 beta: float = 0.0, out: Optional[torch.Tensor] = None, compensation: Optional[torch.Tensor] = None):
    """``alpha * op(a: uint8) @ op(b: int8) + beta * out + compensation`` with int32 accumulation and output."""
    assert a.dtype == torch.uint8 and b.dtype == torch.int8 and a.device.type == "cpu" and b.device.type == "cpu"
    a, b = a.contiguous(), b.contiguous()
    m, k = (a.shape[1], a.shape[0]) if transpose_a else a.shape
    kb, n = (b.shape[1], b.shape[0]) if transpose_b else b.shape
    if k != kb:
        raise ValueError(f"inner dimensions differ: {k} vs {kb}")
    if out is None:
        out = torch.zeros(m, n, dtype=torch.int32)
    if compensation is not None:
        compensation = compensation.to(torch.int32).contiguous()
        assert compensation.shape == (n,)
    rc = _lib.cpu_lib().oslo_cpu_gemm_u8s8s32(
        ctypes.c_int(int(transpose_a)), ctypes.c_int(int(transpose_b)), ctypes.c_longlong(m), ctypes.c_longlong(n),
        ctypes.c_longlong(k), ctypes.c_float(alpha), _ptr(a), ctypes.c_longlong(a.stride(0)), _ptr(b),
        ctypes.c_longlong(b.stride(0)), ctypes.c_float(beta), _ptr(out), ctypes.c_longlong(out.stride(0)), _ptr(compensation))
    if rc:
        raise RuntimeError(f"oslo_cpu_gemm_u8s8s32 failed ({rc})")
    return out


def quantized_linear(x: torch.Tensor, w_q: torch.Tensor, w_clip: float, x_clip: float, bias: Optional[torch.Tensor] = None):
    """``x @ w^T + bias`` on the CPU with int8 arithmetic: ``x`` (fp32 ``[rows, in]``) is quantised symmetrically to int8 with
    ``x_clip`` and stored as uint8 (+128); ``w_q`` is the int8 weight ``[out, in]`` with clip ``w_clip``; the +128 shift is
    undone by the compensation ``-128 * sum_k w_q[:, k]``."""
    xq = torch.round(x.clamp(-x_clip, x_clip) * (127.0 / x_clip)).to(torch.int16)
    xu = (xq + 128).to(torch.uint8)
    comp = -128 * w_q.to(torch.int32).sum(dim=1)
    acc = gemm_u8s8s32(xu, w_q, transpose_b=True, compensation=comp)
    y = acc.float() * (x_clip / 127.0) * (w_clip / 127.0)
    return y if bias is None else y + bias


__all__ = ["sgemm", "gemm_u8s8s32", "quantized_linear"]
