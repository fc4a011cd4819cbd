"""Fused compute + collective kernels over NVLink peer memory (``csrc/fused_collectives_sm100a.cu``).

``available(x, w)`` tells the tensor-parallel ops whether the fused path can run for these operands: CUDA
bf16/fp16 tensors, the symmetric-memory runtime initialised for the tensor group, aligned shapes.  When it
returns False the callers use the NCCL collective + GEMM composition, which is also the correctness oracle
of the fused kernels.
"""
from __future__ import annotations

import torch

_runtime = None  # set by oslo_b200.distributed.symm.enable(...)


def set_runtime(rt):
    global _runtime
    _runtime = rt


def runtime():
    return _runtime


def available(x: torch.Tensor, w: torch.Tensor, kind: str = "any") -> bool:
    """``kind``: "ag" (x is a token shard), "rs" (x holds all tokens) or "any"."""
    rt = _runtime
    if rt is None or not x.is_cuda or x.dim() != 2:
        return False
    if kind == "ag":
        return rt.ws.ag_ok(x, w)
    if kind == "rs":
        return rt.ws.rs_ok(x, w)
    return rt.supports(x, w)


def ag_gemm(x_shard, weight, pc, bias=None):
    """``(all_gather(x_shard) @ weight^T (+ bias), all_gather(x_shard))`` in one kernel."""
    return _runtime.ag_gemm(x_shard, weight, bias)


def gemm_rs(x, weight, pc, addend=None):
    """``reduce_scatter(x @ weight^T + addend)`` over the token dim in one kernel (``addend``: optional local [T, N])."""
    return _runtime.gemm_rs(x, weight, addend=addend)
