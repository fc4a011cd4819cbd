"""LayerNorm / RMSNorm autograd functions backed by ``csrc/norm_sm100a.cu``.

CUDA path for fp32/fp16/bf16 inputs with hidden % 8 == 0 and hidden <= 16384;
pure-torch path on CPU (also the numerics reference in the tests).  Parameters may
be stored in the input dtype or in fp32 ("mixed" variants).

Parity: oslo/torch/nn/modules/functional.py:87-284 (autograd wrappers of the apex kernels).
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _cuda_ok(x, weight):
    if not (x.is_cuda and _lib.has_cuda_kernels()):
        return False
    if x.dtype not in _DT:
        return False
    h = x.shape[-1]
    if h % 8 or h > 16384:
        return False
    if weight is not None and weight.dtype not in (x.dtype, torch.float32):
        return False
    return True


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, rms):
        h = x.shape[-1]
        x2 = x.reshape(-1, h)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        mean = None if rms else torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        wd = _DT[weight.dtype] if weight is not None else _DT[x.dtype]
        rc = _lib.cuda_lib().oslo_norm_forward(
            _lib.ptr(x2), _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(y), _lib.ptr(mean), _lib.ptr(rstd),
            ctypes.c_int(rows), ctypes.c_int(h), ctypes.c_float(eps), ctypes.c_int(1 if rms else 0),
            ctypes.c_int(_DT[x.dtype]), ctypes.c_int(wd), ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_norm_forward failed ({rc})")
        ctx.save_for_backward(x2, weight, mean, rstd)
        ctx.rms, ctx.has_bias, ctx.shape = rms, bias is not None, x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, gy):
        x2, weight, mean, rstd = ctx.saved_tensors
        h = x2.shape[-1]
        rows = x2.shape[0]
        gy2 = gy.reshape(-1, h)
        if not gy2.is_contiguous():
            gy2 = gy2.contiguous()
        dx = torch.empty_like(x2)
        lib = _lib.cuda_lib()
        need_w = weight is not None and ctx.needs_input_grad[1]
        dgamma = torch.empty_like(weight) if need_w else None
        dbeta = torch.empty_like(weight) if (need_w and ctx.has_bias) else None
        parts = lib.oslo_norm_backward_parts(ctypes.c_int(rows), ctypes.c_int(_lib.num_sms()))
        partials = torch.empty(2 * parts * h, dtype=torch.float32, device=x2.device) if need_w else None
        wd = _DT[weight.dtype] if weight is not None else _DT[x2.dtype]
        rc = lib.oslo_norm_backward(
            _lib.ptr(gy2), _lib.ptr(x2), _lib.ptr(mean), _lib.ptr(rstd), _lib.ptr(weight), _lib.ptr(dx),
            _lib.ptr(dgamma), _lib.ptr(dbeta), _lib.ptr(partials), ctypes.c_int(rows), ctypes.c_int(h),
            ctypes.c_int(1 if ctx.rms else 0), ctypes.c_int(_DT[x2.dtype]), ctypes.c_int(wd),
            ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_norm_backward failed ({rc})")
        return dx.view(ctx.shape), dgamma, dbeta, None, None


def layer_norm(x, normalized_shape, weight=None, bias=None, eps: float = 1e-5):
    if isinstance(normalized_shape, int):
        normalized_shape = (normalized_shape,)
    if len(normalized_shape) == 1 and _cuda_ok(x, weight):
        return _NormFn.apply(x, weight, bias, eps, False)
    return F.layer_norm(x, tuple(normalized_shape), weight, bias, eps)


def rms_norm_reference(x, weight, eps):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    return y.to(x.dtype if weight is None else torch.promote_types(x.dtype, weight.dtype) if weight.dtype != torch.float32 else x.dtype)


def rms_norm(x, normalized_shape, weight=None, eps: float = 1e-6):
    if isinstance(normalized_shape, int):
        normalized_shape = (normalized_shape,)
    if len(normalized_shape) == 1 and _cuda_ok(x, weight):
        return _NormFn.apply(x, weight, None, eps, True)
    return rms_norm_reference(x, weight, eps)
