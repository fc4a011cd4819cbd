"""Ring self-attention primitives over the SEQUENCE group.

``RingQK``: each rank holds ``q, k`` of shape ``[b*heads, s/sp, d]`` and obtains
its rows of the full score matrix ``[b*heads, s/sp, s]``.  ``RingAV``: given
probabilities ``[b*heads, s/sp, s]`` and local ``v`` it returns ``[b*heads, s/sp, d]``.
K (or V) blocks circulate ``sp-1`` hops; the receive of hop ``i+1`` is posted
before the matmul of hop ``i`` so transfer and compute overlap (the reference
synchronises the device after every hop, ``_ring_self_attention.py:60-65``).

Parity: ``oslo/torch/distributed/nn/_ring_self_attention.py:70-280``.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .parallel_mode import ParallelMode


def _ring_exchange(send: torch.Tensor, pc):
    """Post send-to-next / recv-from-prev; return (recv_buffer, works)."""
    recv = torch.empty_like(send)
    nxt = pc.get_next_global_rank(ParallelMode.SEQUENCE)
    prv = pc.get_prev_global_rank(ParallelMode.SEQUENCE)
    group = pc.get_group(ParallelMode.SEQUENCE)
    ops = [dist.P2POp(dist.isend, send, nxt, group), dist.P2POp(dist.irecv, recv, prv, group)]
    rank = pc.get_local_rank(ParallelMode.SEQUENCE)
    if rank % 2:
        ops.reverse()
    return recv, dist.batch_isend_irecv(ops)


def _wait(works):
    for w in works:
        w.wait()


class RingQK(torch.autograd.Function):
    @staticmethod
    def forward(ctx, sub_q, sub_k, pc):
        ctx.pc = pc
        ctx.save_for_backward(sub_q, sub_k)
        sp = pc.get_world_size(ParallelMode.SEQUENCE)
        rank = pc.get_local_rank(ParallelMode.SEQUENCE)
        bh, sl, _ = sub_q.shape
        scores = sub_q.new_empty(bh, sl, sl * sp)
        block = sub_k.contiguous()
        for hop in range(sp):
            owner = (rank - hop) % sp
            nxt, works = (None, None)
            if hop < sp - 1:
                nxt, works = _ring_exchange(block, pc)
            torch.matmul(sub_q, block.transpose(1, 2), out=scores[:, :, owner * sl : (owner + 1) * sl])
            if works is not None:
                _wait(works)
                block = nxt
        return scores

    @staticmethod
    def backward(ctx, grad):
        sub_q, sub_k = ctx.saved_tensors
        pc = ctx.pc
        sp = pc.get_world_size(ParallelMode.SEQUENCE)
        rank = pc.get_local_rank(ParallelMode.SEQUENCE)
        sl = sub_q.shape[1]
        # dK[all positions] = gradᵀ · q, summed over ranks, keep own slice
        grad_k_full = torch.matmul(grad.transpose(1, 2), sub_q)
        if sp > 1:
            dist.all_reduce(grad_k_full, group=pc.get_group(ParallelMode.SEQUENCE))
        grad_k = grad_k_full[:, rank * sl : (rank + 1) * sl].contiguous()
        # dQ = Σ_owner grad[:, :, owner] · k_owner : ring K again
        grad_q = torch.zeros_like(sub_q)
        block = sub_k.contiguous()
        for hop in range(sp):
            owner = (rank - hop) % sp
            nxt, works = (None, None)
            if hop < sp - 1:
                nxt, works = _ring_exchange(block, pc)
            grad_q += torch.matmul(grad[:, :, owner * sl : (owner + 1) * sl], block)
            if works is not None:
                _wait(works)
                block = nxt
        return grad_q, grad_k, None


class RingAV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, attn, sub_v, pc):
        ctx.pc = pc
        ctx.save_for_backward(attn, sub_v)
        sp = pc.get_world_size(ParallelMode.SEQUENCE)
        rank = pc.get_local_rank(ParallelMode.SEQUENCE)
        sl = sub_v.shape[1]
        out = torch.zeros(attn.shape[0], attn.shape[1], sub_v.shape[2], dtype=sub_v.dtype, device=sub_v.device)
        block = sub_v.contiguous()
        for hop in range(sp):
            owner = (rank - hop) % sp
            nxt, works = (None, None)
            if hop < sp - 1:
                nxt, works = _ring_exchange(block, pc)
            out += torch.matmul(attn[:, :, owner * sl : (owner + 1) * sl], block)
            if works is not None:
                _wait(works)
                block = nxt
        return out

    @staticmethod
    def backward(ctx, grad):
        attn, sub_v = ctx.saved_tensors
        pc = ctx.pc
        sp = pc.get_world_size(ParallelMode.SEQUENCE)
        rank = pc.get_local_rank(ParallelMode.SEQUENCE)
        sl = sub_v.shape[1]
        grad_v_full = torch.matmul(attn.transpose(1, 2), grad)
        if sp > 1:
            dist.all_reduce(grad_v_full, group=pc.get_group(ParallelMode.SEQUENCE))
        grad_v = grad_v_full[:, rank * sl : (rank + 1) * sl].contiguous()
        grad_attn = torch.empty_like(attn)
        block = sub_v.contiguous()
        for hop in range(sp):
            owner = (rank - hop) % sp
            nxt, works = (None, None)
            if hop < sp - 1:
                nxt, works = _ring_exchange(block, pc)
            torch.matmul(grad, block.transpose(1, 2), out=grad_attn[:, :, owner * sl : (owner + 1) * sl])
            if works is not None:
                _wait(works)
                block = nxt
        return grad_attn, grad_v, None
