"""Vocab-parallel embedding whose forward reads rows from the owning rank's shard over NVLink (``csrc/embedding_sm100a.cu``).

The weight shard must live in symmetric memory (``symm.rehome_parameter``).  Backward is the adjoint composition:
all-gather of the token ids and of the output gradient over the group, then a local scatter-add into this rank's rows.
"""
from __future__ import annotations

import ctypes

import torch

from oslo_b200.distributed import comm

from . import _lib


class _EmbedPull(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, sbuf, pc, mode):
        world = pc.get_world_size(mode)
        v_local, h = weight.shape
        flat = ids.reshape(-1).to(torch.int64).contiguous()
        out = torch.empty(flat.numel(), h, dtype=weight.dtype, device=weight.device)
        sbuf.barrier()  # every rank's table holds this step's weights (the optimizer has finished everywhere)
        rc = _lib.cuda_lib().oslo_embed_pull(_lib.ptr(flat), sbuf.peer_array(0), _lib.ptr(out), ctypes.c_int(flat.numel()),
                                             ctypes.c_int(h * weight.element_size()), ctypes.c_longlong(v_local),
                                             ctypes.c_int(world), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_embed_pull failed ({rc})")
        ctx.save_for_backward(flat)
        ctx.meta = (pc, mode, v_local, h, weight.dtype)
        return out.view(*ids.shape, h)

    @staticmethod
    def backward(ctx, g):
        (flat,) = ctx.saved_tensors
        pc, mode, v_local, h, dtype = ctx.meta
        rank = pc.get_local_rank(mode)
        g2 = g.reshape(-1, h).contiguous()
        all_ids = comm.all_gather(flat, dim=0, parallel_context=pc, parallel_mode=mode)
        all_g = comm.all_gather(g2, dim=0, parallel_context=pc, parallel_mode=mode)
        local = all_ids - rank * v_local
        mine = (local >= 0) & (local < v_local)
        # masked scatter-add without boolean indexing (which would synchronise with the host and cannot be captured
        # in a CUDA graph): rows of other ranks' vocabulary add zeros to row 0
        gw = torch.zeros(v_local, h, dtype=torch.float32, device=g.device)
        gw.index_add_(0, local.clamp(0, v_local - 1), all_g.float() * mine.unsqueeze(1))
        return None, gw.to(dtype), None, None, None


def embedding_pull(ids, weight, sbuf, pc, mode):
    """``out[t] = table[ids[t]]`` where ``table`` is the concatenation of every rank's ``weight`` shard."""
    return _EmbedPull.apply(ids, weight, sbuf, pc, mode)
