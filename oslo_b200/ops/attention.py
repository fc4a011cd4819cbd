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


class DecodeCache:
    """Keys and values of the tokens a model has already seen, for incremental decoding.

    While a cache is active (``with decode_cache(cache):``) every attention call of a forward pass appends the keys and
    values of the tokens it was given to its own slot (slots are taken in call order, one per attention layer) and
    attends over everything stored so far; ``offset`` is the number of tokens stored before the current forward, which
    the models add to their position ids / rotary positions.  ``advance(n)`` is called after each forward.
    Replaces the per-step re-run of the whole prefix; LightSeq keeps the same state in its decoder's cache buffers
    (oslo/lightseq2/inference/model/decoder.cc.cu, gpt_encoder.cc.cu)."""

    def __init__(self):
        self.k, self.v = [], []
        self.offset = 0
        self._layer = 0

    def begin_forward(self):
        self._layer = 0

    def advance(self, n: int):
        self.offset += n

    def reorder(self, index: torch.Tensor):
        """Beam search: hypothesis ``i`` continues hypothesis ``index[i]``."""
        self.k = [t.index_select(0, index) for t in self.k]
        self.v = [t.index_select(0, index) for t in self.v]

    def append(self, k, v):
        i = self._layer
        self._layer += 1
        if i == len(self.k):
            self.k.append(k)
            self.v.append(v)
        else:
            self.k[i] = torch.cat([self.k[i], k], dim=1)
            self.v[i] = torch.cat([self.v[i], v], dim=1)
        return self.k[i], self.v[i]


_CACHE: Optional[DecodeCache] = None


class decode_cache:
    """Context manager that makes ``cache`` the active :class:`DecodeCache` (inference only)."""

    def __init__(self, cache: DecodeCache):
        self.cache = cache

    def __enter__(self):
        global _CACHE
        self.prev, _CACHE = _CACHE, self.cache
        return self.cache

    def __exit__(self, *exc):
        global _CACHE
        _CACHE = self.prev


def decode_offset() -> int:
    """Tokens already held by the active decode cache (0 without one): the position of the first new token."""
    return _CACHE.offset if _CACHE is not None else 0


def _cached_attention(q, k, v, scale, mask=None):
    """New queries ``[b, s, h, d]`` against all stored keys; query ``i`` sees keys up to its own position."""
    K, V = _CACHE.append(k, v)
    b, s, nh, hd = q.shape
    S = K.shape[1]
    scores = torch.einsum("bqhd,bkhd->bhqk", q.float(), K.float()) * scale
    if s > 1:
        qpos = torch.arange(S - s, S, device=q.device).unsqueeze(1)
        scores = scores.masked_fill(torch.arange(S, device=q.device).unsqueeze(0) > qpos, float("-inf"))
    if mask is not None:
        scores = scores + mask[..., -s:, :S].float()
    p = torch.softmax(scores, dim=-1)
    return torch.einsum("bhqk,bkhd->bqhd", p, V.float()).to(q.dtype).reshape(b, s, nh * hd)


def attention(q, k, v, causal: bool = True, scale: Optional[float] = None, mask=None):
    """Multi-head attention.  q, k, v: ``[b, s, heads, head_dim]``; returns ``[b, s, heads*head_dim]``."""
    b, s, nh, hd = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    if _CACHE is not None and causal and not torch.is_grad_enabled():
        return _cached_attention(q, k, v, scale, mask)
    if mask is None and flash_supported(q, k, v):
        return _FlashAttentionFn.apply(q, k, v, causal, float(scale))
    if mask is None and supported(q, k) and s % 8 == 0 and hd % 8 == 0 and k.shape[1] == s:
        return _AttentionFn.apply(q, k, v, causal, float(scale))
    return attention_reference(q, k, v, causal, scale, mask)


# ------------------------------------------------------------------ fused forward
def flash_supported(q, k, v) -> bool:
    b, s, nh, hd = q.shape
    return (supported(q, k) and hd in (64, 128) and s % 128 == 0 and k.shape == q.shape and v.shape == q.shape
            and q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1)


#: one-pass forward with two query tiles per CTA taking turns on the tensor cores (``csrc/attention_pingpong_sm100a.cu``)
#: for sequence lengths that are multiples of 256 (measured 1.2 - 1.3x the two-pass kernel); OSLO_B200_ATTN_PINGPONG=0 keeps
#: the two-pass kernel everywhere
PINGPONG = __import__("os").environ.get("OSLO_B200_ATTN_PINGPONG", "1") == "1"


def flash_attention_forward(q, k, v, causal: bool, scale: float, pingpong=None):
    """Fused attention forward: returns ``(out [b, s, heads*hd], lse [b, heads, s])``.
    q, k, v are ``[b, s, heads, hd]`` views (any token / head / batch strides, unit stride on ``hd``).  ``pingpong`` picks the
    one-pass kernel (``csrc/attention_pingpong_sm100a.cu``, needs ``s % 256 == 0``) over the two-pass kernel
    (``csrc/attention_sm100a.cu``); ``None`` follows :data:`PINGPONG`."""
    import ctypes

    b, s, nh, hd = q.shape
    out = torch.empty(b, s, nh, hd, dtype=q.dtype, device=q.device)
    lse = torch.empty(b, nh, s, dtype=torch.float32, device=q.device)
    st = lambda t: (ctypes.c_longlong(t.stride(1)), ctypes.c_longlong(t.stride(2)), ctypes.c_longlong(t.stride(0)))
    if pingpong is None:
        pingpong = PINGPONG
    if pingpong and s % 256 == 0:
        rc = _lib.cuda_lib().oslo_attention_forward_pingpong(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), _lib.ptr(lse), ctypes.c_int(b), ctypes.c_int(s),
            ctypes.c_int(nh), ctypes.c_int(hd), *st(q), *st(k), *st(v), *st(out), ctypes.c_float(scale),
            ctypes.c_int(1 if causal else 0), ctypes.c_int(1 if q.dtype == torch.bfloat16 else 0),
            _lib.ptr(_lib.status_word(q.device)), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_attention_forward_pingpong failed ({rc})")
        return out.view(b, s, nh * hd), lse
    rc = _lib.cuda_lib().oslo_attention_forward(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), _lib.ptr(lse), ctypes.c_int(b), ctypes.c_int(s), ctypes.c_int(nh),
        ctypes.c_int(hd), *st(q), *st(k), *st(v), *st(out), ctypes.c_float(scale), ctypes.c_int(1 if causal else 0),
        ctypes.c_int(1 if q.dtype == torch.bfloat16 else 0), _lib.ptr(_lib.status_word(q.device)), _lib.stream_ptr())
    if rc:
        raise RuntimeError(f"oslo_attention_forward failed ({rc})")
    return out.view(b, s, nh * hd), lse


def set_backward_groups(groups: int, dq_groups: Optional[int] = None) -> None:
    """1 or 2 element-wise warp groups in the dK / dV kernel of the fused attention backward (2: consecutive query tiles
    alternate between two groups of four warps and the probabilities are double-buffered) and, with ``dq_groups``, in the
    dQ kernel (2: the two groups split every key tile by columns)."""
    rc = _lib.cuda_lib().oslo_attention_backward_set_groups(int(groups))
    if rc:
        raise ValueError("groups must be 1 or 2")
    if dq_groups is not None and _lib.cuda_lib().oslo_attention_backward_set_dq_groups(int(dq_groups)):
        raise ValueError("dq_groups must be 1 or 2")


def flash_attention_backward(q, k, v, out, d_out, lse, dq, dk, dv, causal: bool, scale: float):
    """Fused attention backward (``csrc/attention_bwd_sm100a.cu``).  All tensors ``[b, s, heads, hd]`` views; ``dq, dk, dv``
    are written (they may be slices of one fused buffer)."""
    import ctypes

    b, s, nh, hd = q.shape
    delta = torch.empty(b, nh, s, dtype=torch.float32, device=q.device)
    strides = []
    for t in (q, k, v, out, d_out, dq, dk, dv):
        assert t.stride(-1) == 1
        strides += [t.stride(1), t.stride(2), t.stride(0)]
    arr = (ctypes.c_longlong * len(strides))(*strides)
    rc = _lib.cuda_lib().oslo_attention_backward(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), _lib.ptr(d_out), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv),
        _lib.ptr(lse), _lib.ptr(delta), ctypes.c_int(b), ctypes.c_int(s), ctypes.c_int(nh), ctypes.c_int(hd), arr,
        ctypes.c_float(scale), ctypes.c_int(1 if causal else 0), ctypes.c_int(1 if q.dtype == torch.bfloat16 else 0),
        _lib.ptr(_lib.status_word(q.device)), _lib.stream_ptr())
    if rc:
        raise RuntimeError(f"oslo_attention_backward failed ({rc})")


class _FlashAttentionFn(torch.autograd.Function):
    """Fused forward + backward on separate q, k, v tensors."""

    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        out, lse = flash_attention_forward(q, k, v, causal, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal, ctx.scale = causal, scale
        return out

    @staticmethod
    def backward(ctx, go):
        q, k, v, out, lse = ctx.saved_tensors
        b, s, nh, hd = q.shape
        dqkv = torch.empty(3, b, s, nh, hd, dtype=q.dtype, device=q.device)
        flash_attention_backward(q, k, v, out.view(b, s, nh, hd), go.contiguous().view(b, s, nh, hd), lse, dqkv[0], dqkv[1],
                                 dqkv[2], ctx.causal, ctx.scale)
        return dqkv[0], dqkv[1], dqkv[2], None, None


# ------------------------------------------------------------- fused-QKV entry point
def _split_qkv(qkv5, layout):
    """q, k, v views ``[b, s, heads, hd]`` of a fused projection viewed ``[b, s, heads, 3, hd]`` ("h3d", GPT-NeoX)
    or ``[b, s, 3, heads, hd]`` ("3hd", GPT-2)."""
    if layout == "h3d":
        return qkv5[..., 0, :], qkv5[..., 1, :], qkv5[..., 2, :]
    return qkv5[:, :, 0], qkv5[:, :, 1], qkv5[:, :, 2]


class _QKVAttentionFn(torch.autograd.Function):
    """Rotary embedding (optional) + attention on a fused QKV activation.

    The rotation is applied in place on the projection output, and backward writes dQ / dK / dV straight into
    one buffer with the layout of the input, so no gradient is ever re-assembled by slicing.

    The in-place rotation is deliberately not declared to autograd (``mark_dirty`` would force a second output
    and forbid view inputs): the projection output has no other consumer, and the linear that produced it does
    not keep it for its own backward.
    """

    @staticmethod
    def forward(ctx, qkv, heads, hd, layout, causal, scale, rope):
        from .softmax import _rope_launch

        b, s = qkv.shape[0], qkv.shape[1]
        shape5 = (b, s, heads, 3, hd) if layout == "h3d" else (b, s, 3, heads, hd)
        qkv5 = qkv.view(shape5)
        q, k, v = _split_qkv(qkv5, layout)
        if rope is not None:
            cos, sin, rot, neox = rope
            # q and k lie a fixed distance apart inside the fused buffer: one launch rotates both
            _rope_launch(_tok_view(q), cos, sin, rot, neox, None, False, parts=2, part_stride=k.storage_offset() - q.storage_offset())
        if flash_supported(q, k, v):
            # fused kernel: scores never leave the SM; only the row log-sum-exp is kept for backward
            out, lse = flash_attention_forward(q, k, v, causal, scale)
            ctx.save_for_backward(qkv, lse, out)
            ctx.flash = True
        else:
            qh, kh, vh = (t.permute(0, 2, 1, 3) for t in (q, k, v))
            p = torch.empty(b, heads, s, s, dtype=qkv.dtype, device=qkv.device)
            gemm(qh, kh, out=p, causal=1 if causal else 0)
            softmax_inplace_(p, scale, causal)
            out = torch.empty(b, s, heads * hd, dtype=qkv.dtype, device=qkv.device)
            gemm(p, vh.transpose(-1, -2), out=out.view(b, s, heads, hd).permute(0, 2, 1, 3), causal=2 if causal else 0)
            ctx.save_for_backward(qkv, p)
            ctx.flash = False
        ctx.meta = (heads, hd, layout, causal, scale, rope)
        return out

    @staticmethod
    def backward(ctx, go):
        from .softmax import _rope_launch

        heads, hd, layout, causal, scale, rope = ctx.meta
        if ctx.flash:
            qkv, lse, out_saved = ctx.saved_tensors
        else:
            qkv, p = ctx.saved_tensors
        b, s = qkv.shape[0], qkv.shape[1]
        shape5 = (b, s, heads, 3, hd) if layout == "h3d" else (b, s, 3, heads, hd)
        q, k, v = _split_qkv(qkv.view(shape5), layout)
        if ctx.flash:
            dqkv = torch.empty_like(qkv)
            dq, dk, dv = _split_qkv(dqkv.view(shape5), layout)
            flash_attention_backward(q, k, v, out_saved.view(b, s, heads, hd), go.contiguous().view(b, s, heads, hd), lse, dq, dk,
                                     dv, causal, scale)
            if rope is not None:
                cos, sin, rot, neox = rope
                _rope_launch(_tok_view(dq), cos, sin, rot, neox, None, True, parts=2, part_stride=dk.storage_offset() - dq.storage_offset())
            return dqkv, None, None, None, None, None, None
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = _split_qkv(dqkv.view(shape5), layout)
        goh = go.contiguous().view(b, s, heads, hd).permute(0, 2, 1, 3)
        qh, kh, vh = (t.permute(0, 2, 1, 3) for t in (q, k, v))
        gemm(p.transpose(-1, -2), goh.transpose(-1, -2), out=dv.permute(0, 2, 1, 3), causal=3 if causal else 0)
        dp = torch.empty_like(p)
        gemm(goh, vh, out=dp, causal=1 if causal else 0)
        if causal:
            _softmax_bwd_causal(dp, p, scale)
        else:
            softmax_backward_(dp, p, scale)
        gemm(dp, kh.transpose(-1, -2), out=dq.permute(0, 2, 1, 3), causal=2 if causal else 0)
        gemm(dp.transpose(-1, -2), qh.transpose(-1, -2), out=dk.permute(0, 2, 1, 3), causal=3 if causal else 0)
        if rope is not None:
            cos, sin, rot, neox = rope
            for t in (dq, dk):
                _rope_launch(_tok_view(t), cos, sin, rot, neox, None, True)
        return dqkv, None, None, None, None, None, None


def _tok_view(t):
    """``[b, s, heads, hd]`` strided view -> ``[b*s, heads, hd]`` (token stride must be uniform across b)."""
    b, s, heads, hd = t.shape
    assert t.stride(0) == s * t.stride(1), "tokens must be uniformly strided"
    return t.as_strided((b * s, heads, hd), (t.stride(1), t.stride(2), t.stride(3)), t.storage_offset())


def qkv_attention(qkv, heads: int, head_dim: int, layout: str = "h3d", causal: bool = True, scale=None, rope=None,
                  mask=None):
    """Attention on a fused QKV projection ``[b, s, 3 * heads * head_dim]``; returns ``[b, s, heads * head_dim]``.

    ``rope = (cos, sin, rot_dim, neox)`` applies rotary embedding to q and k first (positions 0..s-1).
    """
    from .softmax import apply_rope

    b, s = qkv.shape[0], qkv.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    if _CACHE is not None and causal and not torch.is_grad_enabled():
        shape5 = (b, s, heads, 3, head_dim) if layout == "h3d" else (b, s, 3, heads, head_dim)
        q, k, v = _split_qkv(qkv.view(shape5), layout)
        if rope is not None:
            cos, sin, rot, neox = rope
            pos = (torch.arange(s, device=qkv.device) + _CACHE.offset).repeat(b)
            q = apply_rope(q.contiguous(), cos, sin, rot, neox, positions=pos)
            k = apply_rope(k.contiguous(), cos, sin, rot, neox, positions=pos)
        return _cached_attention(q, k, v, scale, mask)
    if mask is None and qkv.is_cuda and _lib.has_cuda_kernels() and qkv.dtype in (torch.bfloat16, torch.float16) \
            and s % 8 == 0 and head_dim % 8 == 0 and qkv.is_contiguous():
        if rope is not None and qkv.is_leaf:
            qkv = qkv.clone()
        return _QKVAttentionFn.apply(qkv, heads, head_dim, layout, causal, float(scale), rope)
    shape5 = (b, s, heads, 3, head_dim) if layout == "h3d" else (b, s, 3, heads, head_dim)
    q, k, v = _split_qkv(qkv.view(shape5), layout)
    if rope is not None:
        cos, sin, rot, neox = rope
        q = apply_rope(q, cos, sin, rot, neox)
        k = apply_rope(k, cos, sin, rot, neox)
    return attention(q, k, v, causal, scale, mask)
