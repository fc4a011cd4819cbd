"""Expert-parallel dispatch / combine WITHOUT an all-to-all call: token rows are written straight into the owning
rank's expert buffer (peer stores) and expert outputs are read straight from their owner (peer loads), both inside the
routing kernels of ``csrc/moe_sm100a.cu``.

Buffers (per expert group, in symmetric memory, sized for the largest capacity seen): ``xin`` (expert inputs),
``xout`` (expert outputs), ``gout`` (gradient of the expert outputs), ``gin`` (gradient of the expert inputs); all are
laid out ``[local expert][source rank][C]`` rows of ``h``.  Device-side barriers (bounded waits) separate "everybody
has written" from "everybody may read".  The autograd functions below are drop-in replacements for
``dispatch -> all_to_all`` and ``all_to_all -> combine``.
"""
from __future__ import annotations

import ctypes

import torch

from oslo_b200.distributed import ParallelMode, symm
from oslo_b200.ops import _lib

_DT = {torch.float16: 1, torch.bfloat16: 2}


def available(x: torch.Tensor, ep_size: int) -> bool:
    return (ep_size > 1 and ep_size <= 8 and x.is_cuda and x.dtype in _DT and x.shape[-1] % 8 == 0
            and symm.small_ops_enabled())


def _buffers(pc, rows: int, h: int, esz: int):
    nbytes = rows * h * esz
    # the expert-input buffer holds two generations (see PeerDispatch.forward)
    return [symm.group_buffer(pc, ParallelMode.EXPERT, key, nbytes * (2 if key == "moe_xin" else 1))
            for key in ("moe_xin", "moe_xout", "moe_gout", "moe_gin")]


def _view(buf, rows, h, dtype):
    return buf.payload(0, rows * h * torch.empty((), dtype=dtype).element_size(), dtype, (rows, h))


class PeerDispatch(torch.autograd.Function):
    """tokens [S, h], slot [S, K] -> expert inputs [E_local, ep * C, h] on this rank."""

    @staticmethod
    def forward(ctx, tokens, slot, pc, ep, e_local, C):
        rank = pc.get_local_rank(ParallelMode.EXPERT)
        S, h = tokens.shape
        rows = e_local * ep * C
        xin, _, _, gin = _buffers(pc, rows, h, tokens.element_size())
        # Every source writes ALL its slot rows of every destination (zeros where no token owns the slot), so nothing is
        # cleared beforehand, and two generations of the buffer alternate by call parity: a rank can be at most one call
        # ahead of its peers (the barrier below), so writes of call n + 1 never land on rows that a peer still reads from
        # call n.  One barrier per dispatch instead of a clearing pass and two barriers.
        gen = getattr(xin, "moe_generation", 0)
        xin.moe_generation = gen + 1
        off = (gen & 1) * rows * h * tokens.element_size()
        E = e_local * ep
        flat = slot.reshape(-1)
        owner = torch.arange(S, device=slot.device, dtype=torch.int32).repeat_interleave(slot.shape[1])
        inv = torch.full((E * C + 1,), -1, dtype=torch.int32, device=slot.device)
        inv.scatter_(0, torch.where(flat < 0, torch.full_like(flat, E * C), flat).long(), owner)  # dropped tokens go to the spare cell
        rc = _lib.cuda_lib().oslo_moe_dispatch_rows(_lib.ptr(tokens.contiguous()), xin.peer_array(off), ctypes.c_int(ep), _lib.ptr(inv),
                                                    ctypes.c_int(E), ctypes.c_int(h), ctypes.c_int(rank), ctypes.c_int(e_local),
                                                    ctypes.c_int(C), ctypes.c_int(_DT[tokens.dtype]), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_moe_dispatch_rows (peer) failed ({rc})")
        xin.barrier()  # every source has delivered its rows
        ctx.save_for_backward(slot)
        ctx.meta = (pc, ep, e_local, C, rank, S, h)
        nbytes = rows * h * tokens.element_size()
        local = xin.payload(off, nbytes, tokens.dtype, (rows, h))
        # training keeps the expert inputs for the weight gradients beyond the two calls this generation stays intact
        return (local.clone() if torch.is_grad_enabled() else local).view(e_local, ep * C, h)

    @staticmethod
    def backward(ctx, g):
        (slot,) = ctx.saved_tensors
        pc, ep, e_local, C, rank, S, h = ctx.meta
        rows = e_local * ep * C
        _, _, _, gin = _buffers(pc, rows, h, g.element_size())
        _view(gin, rows, h, g.dtype).copy_(g.reshape(rows, h))
        gin.barrier()  # every owner has published the gradient of its expert inputs
        dx = torch.empty(S, h, dtype=g.dtype, device=g.device)
        rc = _lib.cuda_lib().oslo_moe_pull(gin.peer_array(0), ctypes.c_int(ep), None, _lib.ptr(slot), _lib.ptr(dx), ctypes.c_int(S),
                                           ctypes.c_int(slot.shape[1]), ctypes.c_int(h), ctypes.c_int(rank), ctypes.c_int(e_local),
                                           ctypes.c_int(C), ctypes.c_int(_DT[g.dtype]), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_moe_pull failed ({rc})")
        gin.barrier()  # everybody has read: the buffer may be reused
        return dx, None, None, None, None, None


class PeerCombine(torch.autograd.Function):
    """expert outputs [E_local, ep * C, h] (on their owner), gate weights [S, K], slot [S, K] -> tokens [S, h]."""

    @staticmethod
    def forward(ctx, xout, weight, slot, pc, ep, e_local, C):
        rank = pc.get_local_rank(ParallelMode.EXPERT)
        h = xout.shape[-1]
        rows = e_local * ep * C
        S, K = slot.shape
        _, bout, _, _ = _buffers(pc, rows, h, xout.element_size())
        _view(bout, rows, h, xout.dtype).copy_(xout.reshape(rows, h))
        bout.barrier()  # every owner has published its expert outputs
        w = weight.float().contiguous()
        y = torch.empty(S, h, dtype=xout.dtype, device=xout.device)
        rc = _lib.cuda_lib().oslo_moe_pull(bout.peer_array(0), ctypes.c_int(ep), _lib.ptr(w), _lib.ptr(slot), _lib.ptr(y), ctypes.c_int(S),
                                           ctypes.c_int(K), ctypes.c_int(h), ctypes.c_int(rank), ctypes.c_int(e_local), ctypes.c_int(C),
                                           ctypes.c_int(_DT[xout.dtype]), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_moe_pull failed ({rc})")
        bout.barrier()
        ctx.save_for_backward(xout, w, slot)
        ctx.meta = (pc, ep, e_local, C, rank, weight.dtype)
        return y

    @staticmethod
    def backward(ctx, gy):
        xout, w, slot = ctx.saved_tensors
        pc, ep, e_local, C, rank, wdtype = ctx.meta
        h = xout.shape[-1]
        rows = e_local * ep * C
        S, K = slot.shape
        _, bout, gout, _ = _buffers(pc, rows, h, xout.element_size())
        _view(bout, rows, h, xout.dtype).copy_(xout.reshape(rows, h))  # owners re-publish the outputs (for d weight)
        glocal = _view(gout, rows, h, xout.dtype)
        glocal.zero_()
        gout.barrier()
        dw = torch.empty(S, K, dtype=torch.float32, device=gy.device)
        rc = _lib.cuda_lib().oslo_moe_push_scaled(_lib.ptr(gy.contiguous()), gout.peer_array(0), bout.peer_array(0), ctypes.c_int(ep),
                                                  _lib.ptr(w), _lib.ptr(slot), _lib.ptr(dw), ctypes.c_int(S), ctypes.c_int(K),
                                                  ctypes.c_int(h), ctypes.c_int(rank), ctypes.c_int(e_local), ctypes.c_int(C),
                                                  ctypes.c_int(_DT[xout.dtype]), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_moe_push_scaled failed ({rc})")
        gout.barrier()
        return glocal.clone().view(xout.shape), dw.to(wdtype), None, None, None, None, None
