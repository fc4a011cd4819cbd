"""Fused elementwise ops: bias+GELU, SwiGLU, bias+dropout+residual (``csrc/elementwise_sm100a.cu``).

Parity: oslo/torch/nn/modules/functional.py:23-84,295-298 (TorchScript fusions) and
lightseq2 dropout_kernels.cu (bias+act+dropout, bias+dropout+residual).
"""
from __future__ import annotations

import ctypes
import math

import torch
import torch.nn.functional as F

from . import _lib

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _pack(dtype):
    return 4 if dtype == torch.float32 else 8


def _cuda_ok(x, last_dim=None):
    if not (x.is_cuda and _lib.has_cuda_kernels() and x.dtype in _DT):
        return False
    h = x.shape[-1] if last_dim is None else last_dim
    return h % _pack(x.dtype) == 0


def gelu_tanh_reference(x):
    return F.gelu(x, approximate="tanh")


def colsum(x2: torch.Tensor) -> torch.Tensor:
    """Column sums of a 2-D tensor (bias gradients), fp32 accumulation."""
    if not _cuda_ok(x2):
        return x2.float().sum(0).to(x2.dtype)
    lib = _lib.cuda_lib()
    rows, h = x2.shape
    parts = lib.oslo_colsum_parts(ctypes.c_longlong(rows), ctypes.c_int(_lib.num_sms()))
    partial = torch.empty(parts * h, dtype=torch.float32, device=x2.device)
    out = torch.empty(h, dtype=x2.dtype, device=x2.device)
    rc = lib.oslo_colsum(_lib.ptr(x2), _lib.ptr(out), _lib.ptr(partial), ctypes.c_longlong(rows), ctypes.c_int(h),
                         ctypes.c_int(_DT[x2.dtype]), ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
    if rc:
        raise RuntimeError(f"oslo_colsum failed ({rc})")
    return out


_ACTS = {"gelu_new": 0, "gelu_tanh": 0, "gelu_pytorch_tanh": 0, "gelu_fast": 0, "gelu": 1, "gelu_erf": 1, "relu": 2}


def act_reference(x, act: str):
    code = _ACTS[act]
    if code == 0:
        return gelu_tanh_reference(x)
    return F.gelu(x) if code == 1 else F.relu(x)


class _BiasActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, act):
        xc = x.contiguous()
        y = torch.empty_like(xc)
        h = xc.shape[-1]
        rc = _lib.cuda_lib().oslo_bias_act_forward(
            _lib.ptr(xc), _lib.ptr(bias), _lib.ptr(y), ctypes.c_longlong(xc.numel()), ctypes.c_int(h),
            ctypes.c_int(_DT[xc.dtype]), ctypes.c_int(act), ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_bias_act_forward failed ({rc})")
        ctx.save_for_backward(xc, bias)
        ctx.act = act
        return y

    @staticmethod
    def backward(ctx, gy):
        xc, bias = ctx.saved_tensors
        gy = gy.contiguous()
        dx = torch.empty_like(xc)
        h = xc.shape[-1]
        rc = _lib.cuda_lib().oslo_bias_act_backward(
            _lib.ptr(gy), _lib.ptr(xc), _lib.ptr(bias), _lib.ptr(dx), ctypes.c_longlong(xc.numel()), ctypes.c_int(h),
            ctypes.c_int(_DT[xc.dtype]), ctypes.c_int(ctx.act), ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_bias_act_backward failed ({rc})")
        db = None
        if bias is not None and ctx.needs_input_grad[1]:
            db = colsum(dx.view(-1, h))
        return dx, db, None


def bias_act(x, bias=None, act: str = "gelu_new"):
    """``act(x + bias)`` in one pass; ``act`` is ``gelu_new`` (tanh form), ``gelu`` (erf form) or ``relu``."""
    if act not in _ACTS:
        raise ValueError(f"unsupported activation {act!r}; one of {sorted(_ACTS)}")
    if _cuda_ok(x) and (bias is None or bias.dtype == x.dtype):
        return _BiasActFn.apply(x, bias, _ACTS[act])
    return act_reference(x if bias is None else x + bias, act)


def bias_gelu(x, bias=None):
    """``gelu_tanh(x + bias)``."""
    return bias_act(x, bias, "gelu_new")


fused_bias_gelu = lambda bias, y: bias_gelu(y, bias)  # argument order of the reference's fused_bias_gelu(bias, y)


def fused_gelu(x):
    return bias_gelu(x, None)


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        f = gate_up.shape[-1] // 2
        gu = gate_up.contiguous()
        rows = gu.numel() // (2 * f)
        y = torch.empty(*gu.shape[:-1], f, dtype=gu.dtype, device=gu.device)
        esz = gu.element_size()
        up_ptr = ctypes.c_void_p(gu.data_ptr() + f * esz)
        rc = _lib.cuda_lib().oslo_swiglu_forward(
            _lib.ptr(gu), up_ptr, _lib.ptr(y), ctypes.c_longlong(rows), ctypes.c_int(f), ctypes.c_longlong(2 * f),
            ctypes.c_int(_DT[gu.dtype]), ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_swiglu_forward failed ({rc})")
        ctx.save_for_backward(gu)
        return y

    @staticmethod
    def backward(ctx, gy):
        (gu,) = ctx.saved_tensors
        f = gu.shape[-1] // 2
        rows = gu.numel() // (2 * f)
        gy = gy.contiguous()
        dgu = torch.empty_like(gu)
        esz = gu.element_size()
        rc = _lib.cuda_lib().oslo_swiglu_backward(
            _lib.ptr(gy), _lib.ptr(gu), ctypes.c_void_p(gu.data_ptr() + f * esz), _lib.ptr(dgu),
            ctypes.c_void_p(dgu.data_ptr() + f * esz), ctypes.c_longlong(rows), ctypes.c_int(f),
            ctypes.c_longlong(2 * f), ctypes.c_int(_DT[gu.dtype]), ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_swiglu_backward failed ({rc})")
        return dgu


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for a packed ``[..., 2F]`` tensor (gate first)."""
    f = gate_up.shape[-1] // 2
    if _cuda_ok(gate_up, f):
        return _SwiGLUFn.apply(gate_up)
    gate, up = gate_up[..., :f], gate_up[..., f:]
    return F.silu(gate) * up


_dropout_calls = 0


class _BiasDropoutAddFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, residual, p, seed, offset):
        xc = x.contiguous()
        res = residual.contiguous() if residual is not None else None
        out = torch.empty_like(xc)
        h = xc.shape[-1]
        rc = _lib.cuda_lib().oslo_bias_dropout_add(
            _lib.ptr(xc), _lib.ptr(bias), _lib.ptr(res), _lib.ptr(out), ctypes.c_longlong(xc.numel()), ctypes.c_int(h),
            ctypes.c_float(p), ctypes.c_ulonglong(seed), ctypes.c_ulonglong(offset), ctypes.c_int(0),
            ctypes.c_int(_DT[xc.dtype]), ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_bias_dropout_add failed ({rc})")
        ctx.p, ctx.seed, ctx.offset = p, seed, offset
        ctx.has_bias, ctx.has_res = bias is not None, residual is not None
        return out

    @staticmethod
    def backward(ctx, gy):
        gy = gy.contiguous()
        h = gy.shape[-1]
        if ctx.p > 0:
            dx = torch.empty_like(gy)
            rc = _lib.cuda_lib().oslo_bias_dropout_add(
                _lib.ptr(gy), None, None, _lib.ptr(dx), ctypes.c_longlong(gy.numel()), ctypes.c_int(h),
                ctypes.c_float(ctx.p), ctypes.c_ulonglong(ctx.seed), ctypes.c_ulonglong(ctx.offset), ctypes.c_int(1),
                ctypes.c_int(_DT[gy.dtype]), ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
            if rc:
                raise RuntimeError(f"oslo_bias_dropout_add (bwd) failed ({rc})")
        else:
            dx = gy
        db = colsum(dx.view(-1, h)) if ctx.has_bias and ctx.needs_input_grad[1] else None
        dres = gy if ctx.has_res else None
        return dx, db, dres, None, None, None


def bias_dropout_add(x, bias=None, residual=None, p: float = 0.0, training: bool = True):
    """``residual + dropout(x + bias, p)``; the mask is regenerated in backward from (seed, offset)."""
    global _dropout_calls
    p = float(p) if training else 0.0
    if _cuda_ok(x) and (bias is None or bias.dtype == x.dtype) and (residual is None or residual.dtype == x.dtype):
        # the seed follows the active per-mode generator state, the offset counts dropout calls
        seed = int(torch.cuda.initial_seed()) & 0xFFFFFFFFFFFFFFFF
        offset = 0
        if p > 0:
            _dropout_calls += 1
            offset = _dropout_calls
        return _BiasDropoutAddFn.apply(x, bias, residual, p, seed, offset)
    y = x if bias is None else x + bias
    y = F.dropout(y, p=p, training=training)
    return y if residual is None else residual + y


def fused_bias_dropout(x, bias, p, training, inplace=False):
    return bias_dropout_add(x, bias, None, p, training)


class _SwiGLU2Fn(torch.autograd.Function):
    """``silu(gate) * up`` for two separate tensors (Llama's gate_proj / up_proj outputs)."""

    @staticmethod
    def forward(ctx, gate, up):
        g, u = gate.contiguous(), up.contiguous()
        f = g.shape[-1]
        rows = g.numel() // f
        y = torch.empty_like(g)
        rc = _lib.cuda_lib().oslo_swiglu_forward(
            _lib.ptr(g), _lib.ptr(u), _lib.ptr(y), ctypes.c_longlong(rows), ctypes.c_int(f), ctypes.c_longlong(f),
            ctypes.c_int(_DT[g.dtype]), ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_swiglu_forward failed ({rc})")
        ctx.save_for_backward(g, u)
        return y

    @staticmethod
    def backward(ctx, gy):
        g, u = ctx.saved_tensors
        f = g.shape[-1]
        rows = g.numel() // f
        gy = gy.contiguous()
        dg, du = torch.empty_like(g), torch.empty_like(u)
        rc = _lib.cuda_lib().oslo_swiglu_backward(
            _lib.ptr(gy), _lib.ptr(g), _lib.ptr(u), _lib.ptr(dg), _lib.ptr(du), ctypes.c_longlong(rows), ctypes.c_int(f),
            ctypes.c_longlong(f), ctypes.c_int(_DT[g.dtype]), ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_swiglu_backward failed ({rc})")
        return dg, du


def swiglu2(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    if _cuda_ok(gate) and gate.dtype == up.dtype:
        return _SwiGLU2Fn.apply(gate, up)
    return F.silu(gate) * up
