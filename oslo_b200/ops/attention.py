"""Causal / full multi-head attention on the tcgen05 GEMM kernel plus the fused softmax kernel.

``attention(q, k, v)`` takes ``[b, s, heads, head_dim]`` tensors — strided views into a
fused QKV projection are fine, nothing is copied — and returns ``[b, s, heads * head_dim]``.
The score / probability matrix is materialised in bf16 (``[b, heads, s, s]``); causal
attention skips the tiles above the diagonal in all six products.

Parity: HF GPT-2 ``_attn`` as used by the reference (oslo/transformers/models/gpt2/modeling_gpt2.py:113-165)
and lightseq2 ``SDPALayer`` (csrc/layers_new/sdpa_layer.cpp:10-66).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import _lib
from .gemm import gemm, supported
from .softmax import softmax_backward_, softmax_inplace_, softmax_reference


def attention_reference(q, k, v, causal=True, scale=None, mask=None):
    b, s, nh, hd = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    qf, kf, vf = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    scores = torch.matmul(qf, kf.transpose(-1, -2))
    p = softmax_reference(scores, scale, causal, mask)
    o = torch.matmul(p, vf)
    return o.permute(0, 2, 1, 3).reshape(b, s, nh * hd)


class _AttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        b, s, nh, hd = q.shape
        qh, kh, vh = (t.permute(0, 2, 1, 3) for t in (q, k, v))  # [b, nh, s, hd] views
        p = torch.empty(b, nh, s, s, dtype=q.dtype, device=q.device)
        gemm(qh, kh, out=p, causal=1 if causal else 0)
        softmax_inplace_(p, scale, causal)
        out = torch.empty(b, s, nh, hd, dtype=q.dtype, device=q.device)
        # O = P V : B operand is V^T, i.e. the [s, hd] storage seen MN-major
        gemm(p, vh.transpose(-1, -2), out=out.permute(0, 2, 1, 3), causal=2 if causal else 0)
        ctx.save_for_backward(q, k, v, p)
        ctx.causal, ctx.scale = causal, scale
        return out.view(b, s, nh * hd)

    @staticmethod
    def backward(ctx, go):
        q, k, v, p = ctx.saved_tensors
        b, s, nh, hd = q.shape
        causal, scale = ctx.causal, ctx.scale
        go = go.contiguous().view(b, s, nh, hd)
        goh = go.permute(0, 2, 1, 3)
        qh, kh, vh = (t.permute(0, 2, 1, 3) for t in (q, k, v))
        # one fused gradient buffer [b, s, 3, nh, hd] so the caller's cat/stack is free when q, k, v
        # were slices of one projection
        dqkv = torch.empty(3, b, s, nh, hd, dtype=q.dtype, device=q.device)
        dq, dk, dv = dqkv[0], dqkv[1], dqkv[2]
        # dV = P^T dO
        gemm(p.transpose(-1, -2), goh.transpose(-1, -2), out=dv.permute(0, 2, 1, 3), causal=3 if causal else 0)
        # dP = dO V^T
        dp = torch.empty_like(p)
        gemm(goh, vh, out=dp, causal=1 if causal else 0)
        softmax_backward_(dp, p, scale) if not causal else _softmax_bwd_causal(dp, p, scale)
        # dQ = dS K ; dK = dS^T Q
        gemm(dp, kh.transpose(-1, -2), out=dq.permute(0, 2, 1, 3), causal=2 if causal else 0)
        gemm(dp.transpose(-1, -2), qh.transpose(-1, -2), out=dk.permute(0, 2, 1, 3), causal=3 if causal else 0)
        return dq, dk, dv, None, None


def _softmax_bwd_causal(dp, p, scale):
    # tiles above the diagonal of dp were never written; p is exactly zero there, so clear dp first
    # where p == 0 would multiply garbage: the kernel multiplies by p, and garbage * 0 can be NaN.
    import ctypes

    sq, sk = p.shape[-2], p.shape[-1]
    rc = _lib.cuda_lib().oslo_softmax_backward_causal(
        _lib.ptr(dp), _lib.ptr(p), _lib.ptr(dp), ctypes.c_longlong(p.numel() // sk), ctypes.c_int(sq), ctypes.c_int(sk),
        ctypes.c_float(scale), ctypes.c_int(1 if p.dtype == torch.float16 else 2), ctypes.c_int(_lib.num_sms()),
        _lib.stream_ptr())
    if rc:
        raise RuntimeError(f"oslo_softmax_backward_causal failed ({rc})")
    return dp


def attention(q, k, v, causal: bool = True, scale: Optional[float] = None, mask=None):
    """Multi-head attention.  q, k, v: ``[b, s, heads, head_dim]``; returns ``[b, s, heads*head_dim]``."""
    b, s, nh, hd = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    if mask is None and supported(q, k) and s % 8 == 0 and hd % 8 == 0 and k.shape[1] == s:
        return _AttentionFn.apply(q, k, v, causal, float(scale))
    return attention_reference(q, k, v, causal, scale, mask)
