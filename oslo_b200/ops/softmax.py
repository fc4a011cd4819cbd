"""Scale + mask + softmax (``csrc/elementwise_sm100a.cu``), and rotary embedding.

``scale_mask_softmax(scores, scale, causal, mask)`` handles ``[b, heads, sq, sk]``
or ``[batches, sq, sk]`` scores with an optional additive mask ``[b, 1, 1|sq, sk]``;
the causal variant needs no mask tensor.  Parity: the Megatron fused softmax the
reference declares in oslo/torch/_C/csrc/FusedScaleMaskSoftmaxBinder.cpp:29-127 (its .cu is
missing there) and lightseq2 softmax_kernels.cu.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def softmax_reference(scores, scale=1.0, causal=False, mask=None):
    x = scores.float() * scale
    if mask is not None:
        x = x + mask.float()
    if causal:
        sq, sk = x.shape[-2], x.shape[-1]
        keep = torch.ones(sq, sk, dtype=torch.bool, device=x.device).tril(diagonal=sk - sq)
        x = x.masked_fill(~keep, float("-inf"))
    return torch.softmax(x, dim=-1).to(scores.dtype)


class _SoftmaxFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, scores, scale, causal, mask, inplace):
        x = scores if scores.is_contiguous() else scores.contiguous()
        sq, sk = x.shape[-2], x.shape[-1]
        rows = x.numel() // sk
        y = x if inplace else torch.empty_like(x)
        heads_per_mask, mask_rows, m = 1, 1, None
        if mask is not None:
            m = mask.float().contiguous()
            mask_rows = m.shape[-2]
            batches = x.numel() // (sq * sk)
            heads_per_mask = batches // (m.numel() // (mask_rows * sk))
        rc = _lib.cuda_lib().oslo_softmax_forward(
            _lib.ptr(x), _lib.ptr(y), _lib.ptr(m), ctypes.c_longlong(rows), ctypes.c_int(sq), ctypes.c_int(sk),
            ctypes.c_float(scale), ctypes.c_int(1 if causal else 0), ctypes.c_int(heads_per_mask),
            ctypes.c_int(mask_rows), ctypes.c_int(_DT[x.dtype]), ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_softmax_forward failed ({rc})")
        ctx.save_for_backward(y)
        ctx.scale = scale
        if inplace:
            ctx.mark_dirty(scores)
        return y

    @staticmethod
    def backward(ctx, gy):
        (y,) = ctx.saved_tensors
        gy = gy.contiguous()
        sk = y.shape[-1]
        dx = torch.empty_like(y)
        rc = _lib.cuda_lib().oslo_softmax_backward(
            _lib.ptr(gy), _lib.ptr(y), _lib.ptr(dx), ctypes.c_longlong(y.numel() // sk), ctypes.c_int(sk),
            ctypes.c_float(ctx.scale), ctypes.c_int(_DT[y.dtype]), ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_softmax_backward failed ({rc})")
        return dx, None, None, None, None


def scale_mask_softmax(scores, scale: float = 1.0, causal: bool = False, mask: Optional[torch.Tensor] = None):
    if scores.is_cuda and _lib.has_cuda_kernels() and scores.dtype in (torch.float16, torch.bfloat16) \
            and scores.shape[-1] % 8 == 0:
        return _SoftmaxFn.apply(scores, float(scale), bool(causal), mask, False)
    return softmax_reference(scores, scale, causal, mask)


def softmax_inplace_(scores, scale: float = 1.0, causal: bool = False):
    """No-autograd in-place softmax used by the attention op."""
    sq, sk = scores.shape[-2], scores.shape[-1]
    rc = _lib.cuda_lib().oslo_softmax_forward(
        _lib.ptr(scores), _lib.ptr(scores), None, ctypes.c_longlong(scores.numel() // sk), ctypes.c_int(sq),
        ctypes.c_int(sk), ctypes.c_float(scale), ctypes.c_int(1 if causal else 0), ctypes.c_int(1), ctypes.c_int(1),
        ctypes.c_int(_DT[scores.dtype]), ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
    if rc:
        raise RuntimeError(f"oslo_softmax_forward failed ({rc})")
    return scores


def softmax_backward_(gp, p, scale: float):
    """In place: gp <- scale * p * (gp - sum(gp * p))."""
    sk = p.shape[-1]
    rc = _lib.cuda_lib().oslo_softmax_backward(
        _lib.ptr(gp), _lib.ptr(p), _lib.ptr(gp), ctypes.c_longlong(p.numel() // sk), ctypes.c_int(sk),
        ctypes.c_float(scale), ctypes.c_int(_DT[p.dtype]), ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
    if rc:
        raise RuntimeError(f"oslo_softmax_backward failed ({rc})")
    return gp


# ------------------------------------------------------------------------ rotary
def rope_tables(seq_len: int, rot_dim: int, base: float = 10000.0, device=None):
    inv = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float32, device=device) / rot_dim))
    ang = torch.outer(torch.arange(seq_len, dtype=torch.float32, device=device), inv)
    return ang.cos().contiguous(), ang.sin().contiguous()


def rope_reference(x, cos, sin, rot_dim, neox=True, positions=None, inverse=False):
    """x: [tokens..., heads, head_dim] with the token index as the flattened leading dims modulo seq."""
    shape = x.shape
    hd = shape[-1]
    heads = shape[-2]
    xf = x.reshape(-1, heads, hd).float()
    t = xf.shape[0]
    seq = cos.shape[0]
    pos = positions if positions is not None else torch.arange(t, device=x.device) % seq
    c = cos[pos][:, None, :]
    s = sin[pos][:, None, :]
    if inverse:
        s = -s
    half = rot_dim // 2
    out = xf.clone()
    if neox:
        a, b = xf[..., :half], xf[..., half:rot_dim]
        out[..., :half] = a * c - b * s
        out[..., half:rot_dim] = b * c + a * s
    else:
        a, b = xf[..., 0:rot_dim:2], xf[..., 1:rot_dim:2]
        out[..., 0:rot_dim:2] = a * c - b * s
        out[..., 1:rot_dim:2] = b * c + a * s
    return out.to(x.dtype).view(shape)


def _rope_launch(x, cos, sin, rot_dim, neox, positions, backward, parts: int = 1, part_stride: int = 0):
    # x: [tokens, heads, head_dim] view with unit stride on the last dim; ``parts`` such tensors ``part_stride`` elements
    # apart (q and k of one fused QKV buffer) are rotated by one launch
    tokens, heads, hd = x.shape
    pos = positions.to(torch.int32).contiguous() if positions is not None else None
    rc = _lib.cuda_lib().oslo_rope_parts(
        _lib.ptr(x), _lib.ptr(cos), _lib.ptr(sin), _lib.ptr(pos), ctypes.c_longlong(tokens), ctypes.c_int(heads),
        ctypes.c_int(rot_dim), ctypes.c_int(cos.shape[0]), ctypes.c_longlong(x.stride(0)), ctypes.c_longlong(x.stride(1)),
        ctypes.c_int(parts), ctypes.c_longlong(part_stride), ctypes.c_int(1 if neox else 0), ctypes.c_int(1 if backward else 0),
        ctypes.c_int(_DT[x.dtype]), ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
    if rc:
        raise RuntimeError(f"oslo_rope_parts failed ({rc})")


class _RopeFn(torch.autograd.Function):
    """Rotates in place (the input buffer is the output)."""

    @staticmethod
    def forward(ctx, x, cos, sin, rot_dim, neox, positions):
        ctx.save_for_backward(cos, sin, positions)
        ctx.rot_dim, ctx.neox = rot_dim, neox
        x3 = x.view(-1, x.shape[-2], x.shape[-1]) if x.dim() != 3 else x
        _rope_launch(x3, cos, sin, rot_dim, neox, positions, False)
        ctx.mark_dirty(x)
        return x

    @staticmethod
    def backward(ctx, g):
        cos, sin, positions = ctx.saved_tensors
        g = g.contiguous().clone() if not g.is_contiguous() else g.clone()
        g3 = g.view(-1, g.shape[-2], g.shape[-1])
        _rope_launch(g3, cos, sin, ctx.rot_dim, ctx.neox, positions, True)
        return g, None, None, None, None, None


def apply_rope(x, cos, sin, rot_dim: int, neox: bool = True, positions=None):
    """Rotary embedding on ``x[..., heads, head_dim]``; tokens are the flattened leading dims.

    On CUDA ``x`` must be viewable as ``[tokens, heads, head_dim]`` (strided views of a
    fused QKV buffer are fine) and is rotated in place.
    """
    if x.is_cuda and _lib.has_cuda_kernels() and x.dtype in _DT and x.stride(-1) == 1:
        try:
            x.view(-1, x.shape[-2], x.shape[-1])
            viewable = True
        except RuntimeError:
            viewable = False
        if viewable:
            if x.requires_grad and x.is_leaf:
                x = x.clone()
            return _RopeFn.apply(x, cos, sin, rot_dim, neox, positions)
    return rope_reference(x, cos, sin, rot_dim, neox, positions)
