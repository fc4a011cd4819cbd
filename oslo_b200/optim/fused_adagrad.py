"""Adagrad (optionally with decoupled weight decay), one launch per group.  Parity: oslo/torch/optim/fused_adagrad.py."""
from __future__ import annotations

import ctypes

import torch

from oslo_b200.ops import _lib

from ._base import DT, FusedOptimizerBase


class FusedAdagrad(FusedOptimizerBase):
    def __init__(self, params, lr=1e-2, eps=1e-10, weight_decay=0.0, set_grad_none=True, adagrad_w_mode=False):
        super().__init__(params, dict(lr=lr, eps=eps, weight_decay=weight_decay), set_grad_none)
        self.adagrad_w_mode = 1 if adagrad_w_mode else 0

    @torch.no_grad()
    def step(self, closure=None, noop_flag=None):
        loss = closure() if closure is not None else None
        for gi, group in enumerate(self.param_groups):
            for (cuda, pdt, gdt), ps in self._buckets(group).items():
                for p in ps:
                    if "sum" not in self.state[p]:
                        self.state[p]["sum"] = torch.zeros_like(p, dtype=torch.float32)
                if cuda:
                    t = self._table((gi, pdt, gdt), [[p.data for p in ps], self._grads(ps), [self.state[p]["sum"] for p in ps], None, None])
                    rc = _lib.cuda_lib().oslo_mt_adagrad(
                        _lib.ptr(t.table), _lib.ptr(t.block_map), ctypes.c_int(t.nblocks), ctypes.c_float(group["lr"]),
                        ctypes.c_float(group["eps"]), ctypes.c_float(group["weight_decay"]), ctypes.c_int(self.adagrad_w_mode),
                        _lib.ptr(noop_flag), ctypes.c_int(DT[pdt]), ctypes.c_int(DT[gdt]), _lib.stream_ptr())
                    if rc:
                        raise RuntimeError(f"oslo_mt_adagrad failed ({rc})")
                else:
                    for p in ps:
                        g, pv = p.grad.float(), p.data.float()
                        if not self.adagrad_w_mode:
                            g = g.add(pv, alpha=group["weight_decay"])
                        h = self.state[p]["sum"].addcmul_(g, g)
                        upd = g / (h.sqrt() + group["eps"])
                        if self.adagrad_w_mode:
                            upd = upd.add(pv, alpha=group["weight_decay"])
                        p.data.add_(upd.to(p.dtype), alpha=-group["lr"])
        return loss
