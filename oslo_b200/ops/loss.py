"""Vocab-parallel cross-entropy (``csrc/loss_sm100a.cu``).

``vocab_parallel_cross_entropy(logits, target, parallel_context, ...)`` returns the
per-token loss (fp32, zero where ``target == ignore_index``).  Each TP rank holds the
vocabulary slice ``[rank * V_local, (rank+1) * V_local)`` of the logits.

CUDA path: one pass for the per-row (max, sum-exp, target-logit) triple, ONE exchange
of the triples (all-gather of ``rows x 3`` floats, or direct peer reads when the
symmetric-memory runtime is up), one pass that writes the gradient in place of the
logits — which is then what backward returns (scaled by the incoming gradient).
The reference does three all-reduces and keeps an fp32 softmax
(oslo/torch/nn/modules/loss.py:14-100).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from oslo_b200.distributed import ParallelMode

from . import _lib

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _tp_info(pc, mode):
    if pc is None:
        return 1, 0, None
    return pc.get_world_size(mode), pc.get_local_rank(mode), pc.get_group(mode)


def vocab_parallel_cross_entropy_reference(logits, target, pc=None, mode=ParallelMode.TENSOR_1D, ignore_index=-100,
                                           valid_vocab: Optional[int] = None):
    """Pure-torch implementation with autograd (CPU path and numerics oracle)."""
    world, rank, group = _tp_info(pc, mode)
    v_local = logits.shape[-1]
    start = rank * v_local
    x = logits.float()
    if valid_vocab is not None:
        # columns at or beyond the real vocabulary size are padding: exclude from the softmax
        cols = torch.arange(start, start + v_local, device=x.device)
        x = x.masked_fill(cols >= valid_vocab, float("-inf"))
    return _VPCEFn.apply(x, target, world, start, group, ignore_index)


class _VPCEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, target, world, start, group, ignore_index):
        v_local = x.shape[-1]
        m = x.max(dim=-1).values
        if world > 1:
            dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        e = torch.exp(x - m.unsqueeze(-1))
        s = e.sum(-1)
        local_t = target - start
        in_range = (local_t >= 0) & (local_t < v_local)
        idx = local_t.clamp(0, v_local - 1)
        tv = torch.gather(x, -1, idx.unsqueeze(-1)).squeeze(-1)
        tv = torch.where(in_range, tv, torch.zeros_like(tv))
        if world > 1:
            dist.all_reduce(s, group=group)
            dist.all_reduce(tv, group=group)
        ignored = target == ignore_index
        loss = torch.log(s) + m - tv
        loss = torch.where(ignored, torch.zeros_like(loss), loss)
        soft = e / s.unsqueeze(-1)
        ctx.save_for_backward(soft, idx, in_range, ignored)
        return loss

    @staticmethod
    def backward(ctx, g):
        soft, idx, in_range, ignored = ctx.saved_tensors
        grad = soft.clone()
        sub = in_range.to(grad.dtype)
        grad.scatter_add_(-1, idx.unsqueeze(-1), -sub.unsqueeze(-1))
        g = torch.where(ignored, torch.zeros_like(g), g)
        return grad * g.unsqueeze(-1), None, None, None, None, None


class _VPCECudaFn(torch.autograd.Function):
    """Writes d(loss)/d(logits) into the logits buffer during forward (the logits are consumed).

    The overwrite is not declared to autograd (``mark_dirty`` would add a second output, which autograd forbids
    when the logits are a view, e.g. a reshaped linear output): the logits have no other consumer and the linear
    that produced them does not keep them for its backward.
    """

    @staticmethod
    def forward(ctx, logits, target, pc, mode, ignore_index, valid_vocab):
        world, rank, group = _tp_info(pc, mode)
        v_local = logits.shape[-1]
        x = logits.view(-1, v_local)
        rows = x.shape[0]
        tgt = target.reshape(-1).to(torch.int64).contiguous()
        start = rank * v_local
        valid_local = v_local if valid_vocab is None else max(0, min(v_local, valid_vocab - start))
        lib = _lib.cuda_lib()
        nsm = _lib.num_sms()
        stats = torch.empty(rows, 3, dtype=torch.float32, device=x.device)
        rc = lib.oslo_ce_stats(_lib.ptr(x), _lib.ptr(tgt), _lib.ptr(stats), ctypes.c_int(rows), ctypes.c_int(v_local),
                               ctypes.c_longlong(x.stride(0)), ctypes.c_longlong(start), ctypes.c_int(valid_local),
                               ctypes.c_int(_DT[x.dtype]), ctypes.c_int(nsm), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_ce_stats failed ({rc})")
        from oslo_b200.distributed import symm

        if world > 1 and symm.small_ops_enabled() and world <= 8:
            # ONE exchange without a collective call: the triples are written to symmetric memory, a device-side
            # barrier orders them, and the second kernel reads every peer's triples straight over NVLink
            nbytes = rows * 3 * 4
            buf = symm.group_buffer(pc, mode, "ce_stats", nbytes)
            buf.payload(0, nbytes, torch.float32, (rows, 3)).copy_(stats)
            buf.barrier()  # everybody's triples are in place
            ptrs = [b + buf.payload_offset for b in buf.peer_ptrs]
            gathered = stats
            ce_buf = buf
        elif world > 1:
            gathered = torch.empty(world, rows, 3, dtype=torch.float32, device=x.device)
            dist.all_gather_into_tensor(gathered.view(-1), stats.view(-1), group=group)
            ptrs = [gathered[r].data_ptr() for r in range(world)]
        else:
            gathered = stats
            ptrs = [stats.data_ptr()]
        loss = torch.empty(rows, dtype=torch.float32, device=x.device)
        arr = (ctypes.c_void_p * world)(*ptrs)
        rc = lib.oslo_ce_loss_grad(_lib.ptr(x), _lib.ptr(tgt), arr, ctypes.c_int(world), _lib.ptr(loss), ctypes.c_int(rows),
                                   ctypes.c_int(v_local), ctypes.c_longlong(x.stride(0)), ctypes.c_longlong(start),
                                   ctypes.c_int(valid_local), ctypes.c_longlong(ignore_index), ctypes.c_float(1.0), None,
                                   ctypes.c_int(1), ctypes.c_int(_DT[x.dtype]), ctypes.c_int(nsm), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_ce_loss_grad failed ({rc})")
        if world > 1 and "ce_buf" in locals():
            ce_buf.barrier()  # everybody has read them: the buffer may be overwritten by the next call
        ctx.save_for_backward(logits)  # now holds softmax - onehot
        return loss.view(target.shape)

    @staticmethod
    def backward(ctx, g):
        (grad,) = ctx.saved_tensors
        v = grad.shape[-1]
        g2d = grad.view(-1, v)
        if grad.dtype in (torch.bfloat16, torch.float16) and v % 8 == 0 and g2d.stride(-1) == 1 and g2d.stride(0) % 8 == 0 \
                and g2d.data_ptr() % 16 == 0:
            # one vectorised in-place pass over the vocabulary-sized buffer (the broadcast multiply below runs at a third
            # of the memory bandwidth)
            gs = g.reshape(-1).float().contiguous()
            rc = _lib.cuda_lib().oslo_row_scale(_lib.ptr(g2d), _lib.ptr(gs), ctypes.c_longlong(g2d.shape[0]), ctypes.c_int(v),
                                                ctypes.c_longlong(g2d.stride(0)), ctypes.c_int(1 if grad.dtype == torch.bfloat16 else 0),
                                                ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
            if rc:
                raise RuntimeError(f"oslo_row_scale failed ({rc})")
            return grad, None, None, None, None, None
        g2 = g.reshape(-1, 1).to(grad.dtype)
        out = g2d.mul_(g2).view(grad.shape)
        return out, None, None, None, None, None


def vocab_parallel_cross_entropy(logits, target, parallel_context=None, parallel_mode=ParallelMode.TENSOR_1D,
                                 ignore_index: int = -100, valid_vocab: Optional[int] = None):
    """Per-token loss for vocabulary-sharded ``logits [..., V_local]`` and global ``target [...]``.

    On CUDA the logits tensor is overwritten with its own gradient (it must not be
    used afterwards) so no second vocabulary-sized buffer is ever allocated.
    """
    if logits.is_cuda and _lib.has_cuda_kernels() and logits.dtype in _DT and logits.is_contiguous():
        if logits.is_leaf:
            logits = logits.clone()
        return _VPCECudaFn.apply(logits, target, parallel_context, parallel_mode, ignore_index, valid_vocab)
    return vocab_parallel_cross_entropy_reference(logits, target, parallel_context, parallel_mode, ignore_index, valid_vocab)
