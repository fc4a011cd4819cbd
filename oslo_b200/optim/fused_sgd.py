"""SGD with momentum / Nesterov / weight decay, one kernel launch per group.  Parity: oslo/torch/optim/fused_sgd.py."""
from __future__ import annotations

import ctypes

import torch

from oslo_b200.ops import _lib

from ._base import DT, FusedOptimizerBase


class FusedSGD(FusedOptimizerBase):
    def __init__(self, params, lr, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False, wd_after_momentum=False,
                 set_grad_none=True):
        if nesterov and (momentum <= 0 or dampening != 0):
            raise ValueError("Nesterov momentum requires a momentum and zero dampening")
        super().__init__(params, dict(lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay,
                                      nesterov=nesterov), set_grad_none)
        self.wd_after_momentum = wd_after_momentum

    @torch.no_grad()
    def step(self, closure=None, grad_scale: float = 1.0, noop_flag=None):
        loss = closure() if closure is not None else None
        for gi, group in enumerate(self.param_groups):
            first_run = not group.get("_started", False)
            group["_started"] = True
            for (cuda, pdt, gdt), ps in self._buckets(group).items():
                for p in ps:
                    if group["momentum"] != 0 and "momentum_buffer" not in self.state[p]:
                        self.state[p]["momentum_buffer"] = torch.zeros_like(p, dtype=torch.float32)
                if cuda:
                    bufs = [self.state[p]["momentum_buffer"] for p in ps] if group["momentum"] != 0 else [p.data for p in ps]
                    t = self._table((gi, pdt, gdt), [[p.data for p in ps], self._grads(ps), bufs, None, None])
                    rc = _lib.cuda_lib().oslo_mt_sgd(
                        _lib.ptr(t.table), _lib.ptr(t.block_map), ctypes.c_int(t.nblocks), ctypes.c_float(group["lr"]),
                        ctypes.c_float(group["momentum"]), ctypes.c_float(group["dampening"]),
                        ctypes.c_float(group["weight_decay"]), ctypes.c_float(grad_scale), ctypes.c_int(int(group["nesterov"])),
                        ctypes.c_int(int(first_run)), ctypes.c_int(int(self.wd_after_momentum)), _lib.ptr(noop_flag),
                        ctypes.c_int(DT[pdt]), ctypes.c_int(DT[gdt]), _lib.stream_ptr())
                    if rc:
                        raise RuntimeError(f"oslo_mt_sgd failed ({rc})")
                else:
                    for p in ps:
                        g = p.grad.float() * grad_scale
                        wd, mom = group["weight_decay"], group["momentum"]
                        if wd and not self.wd_after_momentum:
                            g = g.add(p.data.float(), alpha=wd)
                        if mom:
                            buf = self.state[p]["momentum_buffer"]
                            if first_run:
                                buf.copy_(g)
                            else:
                                buf.mul_(mom).add_(g, alpha=1 - group["dampening"])
                            g = g.add(buf, alpha=mom) if group["nesterov"] else buf
                        if wd and self.wd_after_momentum:
                            g = g.add(p.data.float(), alpha=wd)
                        p.data.add_(g.to(p.dtype), alpha=-group["lr"])
        return loss
