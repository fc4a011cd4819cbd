"""NovoGrad: Adam-like first moment on gradients normalised by a per-TENSOR second moment (a blend of squared
gradient norms).  Parity: oslo/torch/optim/fused_novograd.py."""
from __future__ import annotations

import ctypes

import torch

from oslo_b200.ops import _lib
from oslo_b200.ops.multi_tensor import sumsq

from ._base import DT, FusedOptimizerBase


class FusedNovoGrad(FusedOptimizerBase):
    def __init__(self, params, lr=1e-3, bias_correction=True, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                 amsgrad=False, reg_inside_moment=False, grad_averaging=True, norm_type=2, init_zero=False,
                 set_grad_none=True):
        if amsgrad:
            raise RuntimeError("FusedNovoGrad does not support the AMSGrad variant")
        if norm_type != 2:
            raise RuntimeError("FusedNovoGrad supports the L2 norm only")
        super().__init__(params, dict(lr=lr, bias_correction=bias_correction, betas=betas, eps=eps,
                                      weight_decay=weight_decay, grad_averaging=grad_averaging), set_grad_none)
        self.init_zero = init_zero

    @torch.no_grad()
    def step(self, closure=None, noop_flag=None):
        loss = closure() if closure is not None else None
        for gi, group in enumerate(self.param_groups):
            group["step"] = group.get("step", 0) + 1
            step = group["step"]
            b1, b2 = group["betas"]
            beta3 = 1 - b1 if group["grad_averaging"] else 1.0
            bc1 = 1 - b1**step if group["bias_correction"] else 1.0
            bc2 = (1 - b2**step) ** 0.5 if group["bias_correction"] else 1.0
            for (cuda, pdt, gdt), ps in self._buckets(group).items():
                for p in ps:
                    if "exp_avg" not in self.state[p]:
                        self.state[p]["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                key = ("v", gi, cuda, pdt, gdt)
                if cuda:
                    t = self._table((gi, pdt, gdt), [[p.data for p in ps], self._grads(ps), [self.state[p]["exp_avg"] for p in ps], None, None])
                    _, g_sq = sumsq(t, 1, gdt, per_tensor=True)
                    gnorm = g_sq.sqrt()
                else:
                    gnorm = torch.stack([p.grad.float().norm() for p in ps])
                v = group.get(key)
                if v is None or v.numel() != len(ps):
                    v = torch.zeros_like(gnorm) if self.init_zero else gnorm.clone()
                    if self.init_zero:
                        v = (b2 * v.pow(2) + (1 - b2) * gnorm.pow(2)).sqrt()
                else:
                    v = (b2 * v.pow(2) + (1 - b2) * gnorm.pow(2)).sqrt()
                group[key] = v
                if cuda:
                    rc = _lib.cuda_lib().oslo_mt_novograd(
                        _lib.ptr(t.table), _lib.ptr(t.block_map), ctypes.c_int(t.nblocks), ctypes.c_float(group["lr"]),
                        ctypes.c_float(b1), ctypes.c_float(b2), ctypes.c_float(beta3), ctypes.c_float(group["eps"]),
                        ctypes.c_float(group["weight_decay"]), ctypes.c_float(bc1), ctypes.c_float(bc2), ctypes.c_int(1),
                        _lib.ptr(v), _lib.ptr(noop_flag), ctypes.c_int(DT[pdt]), ctypes.c_int(DT[gdt]), _lib.stream_ptr())
                    if rc:
                        raise RuntimeError(f"oslo_mt_novograd failed ({rc})")
                else:
                    for i, p in enumerate(ps):
                        pv = p.data.float()
                        g = p.grad.float() / (v[i] / bc2 + group["eps"]) + group["weight_decay"] * pv
                        m = self.state[p]["exp_avg"].mul_(b1).add_(g, alpha=beta3)
                        p.data.add_((m / bc1).to(p.dtype), alpha=-group["lr"])
        return loss
