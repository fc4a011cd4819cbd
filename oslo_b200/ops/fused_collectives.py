"""Fused compute + collective kernels over NVLink peer memory (``csrc/fused_collectives_sm100a.cu``).

``available(x, w)`` tells the tensor-parallel ops whether the fused path can run for these operands: CUDA
bf16/fp16 tensors, the symmetric-memory runtime initialised for the tensor group, aligned shapes.  When it
returns False the callers use the NCCL collective + GEMM composition, which is also the correctness oracle
of the fused kernels.
"""
from __future__ import annotations

import torch

from oslo_b200.utils.nvtx import annotate

_runtime = None  # the 1-D group's runtime, set by oslo_b200.distributed.symm.enable(...)
_runtimes = {}   # ParallelMode -> runtime, for the groups of the 2-D / 2.5-D / 3-D layouts


def set_runtime(rt, mode=None):
    """Register (or with ``rt=None`` drop) the runtime of one group.  ``mode=None`` or the 1-D tensor mode is the
    runtime that the sequence-parallel linears use."""
    global _runtime
    from oslo_b200.distributed import ParallelMode

    if mode is None or mode == ParallelMode.TENSOR_1D:
        _runtime = rt
    if mode is not None:
        if rt is None:
            _runtimes.pop(mode, None)
        else:
            _runtimes[mode] = rt


def clear_runtimes():
    global _runtime
    _runtime = None
    _runtimes.clear()


def runtime(mode=None):
    return _runtime if mode is None else _runtimes.get(mode)


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


def ag_gemm(x_shard, weight, pc, bias=None, keep=True, gelu_grad_of=None):
    """``(all_gather(x_shard) @ weight^T (+ bias), all_gather(x_shard))`` in one kernel.  ``keep=False`` returns the gathered
    activations as a view of the workspace, valid until two more fused calls have been issued.  ``gelu_grad_of`` (a ``[T, N]``
    pre-activation) multiplies the product by ``gelu'`` of it in the epilogue."""
    with annotate("oslo.ag_gemm"):
        return _runtime.ag_gemm(x_shard, weight, bias, keep, gelu_grad_of)


def gemm_rs(x, weight, pc, addend=None, pair=None):
    """``reduce_scatter(x @ weight^T + addend + pair[0] @ pair[1]^T)`` over the token dim (``addend``: optional local
    ``[T, N]``; ``pair``: an optional second ``(x', weight')`` product that leaves in the same reduce-scatter)."""
    with annotate("oslo.gemm_rs"):
        return _runtime.gemm_rs(x, weight, addend=addend, pair=pair)


def feature_rs_available(x: torch.Tensor, w: torch.Tensor, mode) -> bool:
    """Can ``gemm_rs_features`` run for these operands over the group of ``mode``?"""
    rt = _runtimes.get(mode)
    return rt is not None and x.is_cuda and x.dim() == 2 and rt.ws.rs_ok(x, w, along_n=True)


def gemm_rs_features(x, weight, mode):
    """``reduce_scatter(x @ weight^T)`` over the FEATURE dim within the group of ``mode`` (2-D / 2.5-D linears):
    ``[T, K] x [N, K]^T -> [T, N / q]`` in one kernel."""
    with annotate("oslo.gemm_rs_features"):
        return _runtimes[mode].gemm_rs(x, weight, along_n=True)


def gather_scatter_available(x_shard: torch.Tensor, w: torch.Tensor, ag_mode, rs_mode) -> bool:
    a, r = _runtimes.get(ag_mode), _runtimes.get(rs_mode)
    return a is not None and r is not None and x_shard.is_cuda and x_shard.dim() == 2 and a.ws.ag_rs_ok(r.ws, x_shard, w)


def ag_gemm_rs(x_shard, weight, ag_mode, rs_mode):
    """``(reduce_scatter_rows over rs_mode (all_gather_rows over ag_mode (x_shard) @ weight^T), gathered x)`` in one
    kernel (the 3-D linear: INPUT gather, OUTPUT scatter)."""
    with annotate("oslo.ag_gemm_rs"):
        return _runtimes[ag_mode].ws.ag_gemm_rs(_runtimes[rs_mode].ws, x_shard, weight)
