"""Device-resident tensor tables for the multi-tensor kernels (``csrc/optim_sm100a.cu``).

A :class:`TensorTable` describes N tensors x up to 5 roles (param, grad, exp_avg, ...)
as one int64 device array of records plus a block map, built once and reused while
the data pointers stay the same.  One kernel launch then covers every tensor.

Parity: ``MultiTensorApply`` of the reference (oslo/torch/utils/multi_tensor_apply/*.py), which
re-packs pointer lists into kernel arguments on every call.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import torch

from . import _lib

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


class TensorTable:
    def __init__(self, columns: Sequence[Optional[Sequence[torch.Tensor]]], device=None):
        """``columns[role][i]`` is tensor ``i`` in ``role`` (a column may be None)."""
        lib = _lib.cuda_lib()
        self.chunk = lib.oslo_mt_chunk()
        first = next(c for c in columns if c is not None)
        self.n = len(first)
        self.device = device or first[0].device
        self._key = None
        self.table = None
        self.block_map = None
        self.nblocks = 0
        self.update(columns)

    @staticmethod
    def _ptr_key(columns):
        return tuple(tuple(t.data_ptr() for t in c) if c is not None else None for c in columns)

    def update(self, columns):
        key = self._ptr_key(columns)
        if key == self._key:
            return
        self._key = key
        first = next(c for c in columns if c is not None)
        recs, bmap = [], []
        for i in range(len(first)):
            numel = first[i].numel()
            row = [numel]
            for role in range(5):
                col = columns[role] if role < len(columns) else None
                row.append(col[i].data_ptr() if col is not None else 0)
            recs.append(row)
            for c in range((numel + self.chunk - 1) // self.chunk):
                bmap.append((i, c))
        # staged through pinned memory with async copies: legal while a CUDA graph is being captured (the pinned
        # tensors are kept alive because a replay reads them again)
        host_table = torch.tensor(recs, dtype=torch.int64)
        host_map = torch.tensor(bmap, dtype=torch.int32).reshape(-1, 2)
        if torch.cuda.is_available():
            host_table, host_map = host_table.pin_memory(), host_map.pin_memory()
        self._host = (host_table, host_map)
        self.table = host_table.to(self.device, non_blocking=True)
        self.block_map = host_map.to(self.device, non_blocking=True)
        self.nblocks = len(bmap)
        self.columns = columns  # keep tensors alive


def l2norm(table: TensorTable, which: int, dtype, per_tensor: bool = False, max_norm: bool = False, flag=None):
    """Returns (global_norm, per_tensor_norms or None): L2 (or max) norms of column ``which``."""
    dev = table.device
    g = torch.zeros(1, dtype=torch.float32, device=dev)
    pt = torch.zeros(table.n, dtype=torch.float32, device=dev) if per_tensor else None
    rc = _lib.cuda_lib().oslo_mt_norm(
        _lib.ptr(table.table), _lib.ptr(table.block_map), ctypes.c_int(table.nblocks), ctypes.c_int(which),
        _lib.ptr(g), _lib.ptr(pt), _lib.ptr(flag), ctypes.c_int(1 if max_norm else 0), ctypes.c_int(_DT[dtype]),
        _lib.stream_ptr())
    if rc:
        raise RuntimeError(f"oslo_mt_norm failed ({rc})")
    if max_norm:
        return g, pt
    return g.sqrt_(), (pt.sqrt_() if pt is not None else None)


def sumsq(table: TensorTable, which: int, dtype, per_tensor: bool = False, flag=None):
    """Sum of squares of column ``which`` (global [1] and optionally per tensor)."""
    dev = table.device
    g = torch.zeros(1, dtype=torch.float32, device=dev)
    pt = torch.zeros(table.n, dtype=torch.float32, device=dev) if per_tensor else None
    rc = _lib.cuda_lib().oslo_mt_norm(
        _lib.ptr(table.table), _lib.ptr(table.block_map), ctypes.c_int(table.nblocks), ctypes.c_int(which),
        _lib.ptr(g), _lib.ptr(pt), _lib.ptr(flag), ctypes.c_int(0), ctypes.c_int(_DT[dtype]), _lib.stream_ptr())
    if rc:
        raise RuntimeError(f"oslo_mt_norm failed ({rc})")
    return g, pt


def scale_cast(src: torch.Tensor, dst: torch.Tensor, scale: float = 1.0, dev_scale: Optional[torch.Tensor] = None):
    """``dst = src * scale * dev_scale`` with dtype conversion, one pass."""
    assert src.numel() == dst.numel() and src.is_contiguous() and dst.is_contiguous()
    rc = _lib.cuda_lib().oslo_scale_cast(
        _lib.ptr(src), _lib.ptr(dst), ctypes.c_longlong(src.numel()), ctypes.c_float(scale), _lib.ptr(dev_scale),
        ctypes.c_int(_DT[src.dtype]), ctypes.c_int(_DT[dst.dtype]), ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
    if rc:
        raise RuntimeError(f"oslo_scale_cast failed ({rc})")
    return dst
