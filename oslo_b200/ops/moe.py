"""Index-based mixture-of-experts routing ops (``csrc/moe_sm100a.cu``) with pure-torch fallbacks.

``positions(expert_idx, num_experts)``  rank of every (token, choice) inside its expert's buffer (first choices of all
tokens come before second choices).  ``dispatch(x, slot, rows)`` gathers token rows into the expert buffer;
``combine(buf, weight, slot)`` is the weighted scatter back.  Both are autograd functions.

Parity: ``EPDispatch`` / ``EPCombine`` and ``cumsum_sub_one`` of the reference
(oslo/torch/nn/parallel/expert_parallel/_ops.py:30-103), which its layers never call.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _cuda(x):
    return x.is_cuda and _lib.has_cuda_kernels() and x.dtype in _DT


def positions(expert_idx: torch.Tensor, num_experts: int):
    """``expert_idx [S, K]`` (int, -1 = unrouted) -> ``(pos [S, K] int32, counts [E] int32)``."""
    S, K = expert_idx.shape
    if expert_idx.is_cuda and _lib.has_cuda_kernels():
        idx = expert_idx.to(torch.int32).contiguous()
        pos = torch.zeros(S, K, dtype=torch.int32, device=idx.device)
        counts = torch.empty(num_experts, dtype=torch.int32, device=idx.device)
        rc = _lib.cuda_lib().oslo_moe_positions(_lib.ptr(idx), _lib.ptr(pos), _lib.ptr(counts), ctypes.c_int(S), ctypes.c_int(K),
                                                ctypes.c_int(num_experts), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_moe_positions failed ({rc})")
        return pos, counts
    pos = torch.zeros(S, K, dtype=torch.int32, device=expert_idx.device)
    carry = torch.zeros(num_experts, dtype=torch.long, device=expert_idx.device)
    for k in range(K):
        col = expert_idx[:, k].long()
        valid = col >= 0
        oh = torch.nn.functional.one_hot(col.clamp(min=0), num_experts) * valid.unsqueeze(1)
        before = torch.cumsum(oh, 0) - oh + carry
        pos[:, k] = (before * oh).sum(1).to(torch.int32)
        carry = carry + oh.sum(0)
    return pos, carry.to(torch.int32)


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, slot, rows):
        S, H = x.shape
        K = slot.shape[1]
        buf = torch.zeros(rows, H, dtype=x.dtype, device=x.device)
        ptrs = (ctypes.c_void_p * 1)(buf.data_ptr())
        rc = _lib.cuda_lib().oslo_moe_dispatch(_lib.ptr(x), ptrs, ctypes.c_int(1), _lib.ptr(slot), ctypes.c_int(S), ctypes.c_int(K),
                                               ctypes.c_int(H), ctypes.c_int(0), ctypes.c_int(1), ctypes.c_int(rows),
                                               ctypes.c_int(_DT[x.dtype]), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_moe_dispatch failed ({rc})")
        ctx.save_for_backward(slot)
        return buf

    @staticmethod
    def backward(ctx, gbuf):
        (slot,) = ctx.saved_tensors
        gbuf = gbuf.contiguous()
        S, K = slot.shape
        H = gbuf.shape[1]
        dx = torch.empty(S, H, dtype=gbuf.dtype, device=gbuf.device)
        rc = _lib.cuda_lib().oslo_moe_dispatch_backward(_lib.ptr(gbuf), _lib.ptr(slot), _lib.ptr(dx), ctypes.c_int(S), ctypes.c_int(K),
                                                        ctypes.c_int(H), ctypes.c_int(_DT[gbuf.dtype]), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_moe_dispatch_backward failed ({rc})")
        return dx, None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, buf, weight, slot):
        S, K = slot.shape
        H = buf.shape[1]
        buf = buf.contiguous()
        w = weight.float().contiguous()
        y = torch.empty(S, H, dtype=buf.dtype, device=buf.device)
        rc = _lib.cuda_lib().oslo_moe_combine(_lib.ptr(buf), _lib.ptr(w), _lib.ptr(slot), _lib.ptr(y), ctypes.c_int(S), ctypes.c_int(K),
                                              ctypes.c_int(H), ctypes.c_int(_DT[buf.dtype]), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_moe_combine failed ({rc})")
        ctx.save_for_backward(buf, w, slot)
        ctx.wdtype = weight.dtype
        return y

    @staticmethod
    def backward(ctx, gy):
        buf, w, slot = ctx.saved_tensors
        gy = gy.contiguous()
        S, K = slot.shape
        H = buf.shape[1]
        dbuf = torch.zeros_like(buf)
        dw = torch.empty(S, K, dtype=torch.float32, device=buf.device)
        rc = _lib.cuda_lib().oslo_moe_combine_backward(_lib.ptr(gy), _lib.ptr(buf), _lib.ptr(w), _lib.ptr(slot), _lib.ptr(dbuf),
                                                       _lib.ptr(dw), ctypes.c_int(S), ctypes.c_int(K), ctypes.c_int(H),
                                                       ctypes.c_int(_DT[buf.dtype]), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_moe_combine_backward failed ({rc})")
        return dbuf, dw.to(ctx.wdtype), None


def dispatch(x: torch.Tensor, slot: torch.Tensor, rows: int) -> torch.Tensor:
    """``buf[slot[s, k]] = x[s]`` for slots >= 0; unused rows are zero.  ``x [S, H]``, ``slot [S, K]`` int32."""
    if _cuda(x) and (x.shape[1] * x.element_size()) % 16 == 0:
        return _Dispatch.apply(x.contiguous(), slot.contiguous(), rows)
    S, H = x.shape
    K = slot.shape[1]
    flat = slot.reshape(-1).long()
    valid = flat >= 0
    src = x.unsqueeze(1).expand(S, K, H).reshape(-1, H)
    buf = x.new_zeros(rows, H)
    return buf.index_add(0, flat[valid], src[valid])


def combine(buf: torch.Tensor, weight: torch.Tensor, slot: torch.Tensor) -> torch.Tensor:
    """``y[s] = sum_k weight[s, k] * buf[slot[s, k]]``."""
    if _cuda(buf) and buf.shape[1] % 8 == 0:
        return _Combine.apply(buf, weight, slot.contiguous())
    valid = (slot >= 0)
    rows = buf[slot.clamp(min=0).long()]  # [S, K, H]
    w = (weight * valid).to(buf.dtype).unsqueeze(-1)
    return (rows * w).sum(1)
