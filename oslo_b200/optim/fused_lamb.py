"""LAMB: Adam-style update with global gradient-norm clipping and a per-tensor trust ratio.

Stage 1 (moments + raw update) and stage 2 (``p -= lr * ||p|| / ||u|| * u``) are two launches per group, with the
three norm reductions in between on the same device tables.  ``FusedMixedPrecisionLamb`` reads the GradScaler's
``inv_scale`` / ``found_inf`` device scalars so an overflowing step is skipped without a host sync.
Parity: oslo/torch/optim/fused_lamb.py, fused_mixed_precision_lamb.py.
"""
from __future__ import annotations

import ctypes
import math

import torch

from oslo_b200.ops import _lib
from oslo_b200.ops.multi_tensor import sumsq

from ._base import DT, FusedOptimizerBase


class FusedLamb(FusedOptimizerBase):
    def __init__(self, params, lr=1e-3, bias_correction=True, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.01,
                 amsgrad=False, adam_w_mode=True, grad_averaging=True, set_grad_none=True, max_grad_norm=1.0,
                 use_nvlamb=False):
        if amsgrad:
            raise RuntimeError("FusedLamb does not support the AMSGrad variant")
        super().__init__(params, dict(lr=lr, bias_correction=bias_correction, betas=betas, eps=eps,
                                      weight_decay=weight_decay, grad_averaging=grad_averaging,
                                      max_grad_norm=max_grad_norm), set_grad_none)
        self.adam_w_mode = 1 if adam_w_mode else 0
        self.use_nvlamb = use_nvlamb

    def _global_grad_sumsq(self, inv_scale=None):
        """Sum of squared gradients over every parameter of every group (device scalar on CUDA, float on CPU)."""
        total_dev, total_cpu = None, 0.0
        for gi, group in enumerate(self.param_groups):
            for (cuda, pdt, gdt), ps in self._buckets(group).items():
                if cuda:
                    t = self._table(("n", gi, pdt, gdt), [self._grads(ps), None, None, None, None])
                    g, _ = sumsq(t, 0, gdt)
                    total_dev = g if total_dev is None else total_dev + g
                else:
                    total_cpu += sum(float(p.grad.float().pow(2).sum()) for p in ps)
        return total_dev, total_cpu

    @torch.no_grad()
    def step(self, closure=None, inv_scale=None, noop_flag=None):
        loss = closure() if closure is not None else None
        total_dev, total_cpu = self._global_grad_sumsq()
        for gi, group in enumerate(self.param_groups):
            group["step"] = group.get("step", 0) + 1
            b1, b2 = group["betas"]
            beta3 = 1 - b1 if group["grad_averaging"] else 1.0
            step = group["step"]
            bc1 = 1 - b1**step if group["bias_correction"] else 1.0
            bc2 = 1 - b2**step if group["bias_correction"] else 1.0
            for (cuda, pdt, gdt), ps in self._buckets(group).items():
                for p in ps:
                    st = self.state[p]
                    if "exp_avg" not in st:
                        st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                        st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                        st["update"] = torch.zeros_like(p, dtype=torch.float32)
                if cuda:
                    cols = [[p.data for p in ps], self._grads(ps), [self.state[p]["exp_avg"] for p in ps],
                            [self.state[p]["exp_avg_sq"] for p in ps], [self.state[p]["update"] for p in ps]]
                    t = self._table((gi, pdt, gdt), cols)
                    lib = _lib.cuda_lib()
                    gsum = total_dev if total_cpu == 0.0 else total_dev + total_cpu
                    rc = lib.oslo_mt_lamb_stage1(
                        _lib.ptr(t.table), _lib.ptr(t.block_map), ctypes.c_int(t.nblocks), ctypes.c_float(group["lr"]),
                        ctypes.c_float(b1), ctypes.c_float(b2), ctypes.c_float(beta3), ctypes.c_float(group["eps"]),
                        ctypes.c_float(group["weight_decay"]), ctypes.c_float(bc1), ctypes.c_float(bc2),
                        ctypes.c_float(group["max_grad_norm"]), ctypes.c_int(self.adam_w_mode), ctypes.c_int(int(self.use_nvlamb)),
                        _lib.ptr(gsum), _lib.ptr(inv_scale), _lib.ptr(noop_flag), ctypes.c_int(DT[pdt]), ctypes.c_int(DT[gdt]),
                        _lib.stream_ptr())
                    if rc:
                        raise RuntimeError(f"oslo_mt_lamb_stage1 failed ({rc})")
                    _, p_sq = sumsq(t, 0, pdt, per_tensor=True)
                    _, u_sq = sumsq(t, 4, torch.float32, per_tensor=True)
                    rc = lib.oslo_mt_lamb_stage2(
                        _lib.ptr(t.table), _lib.ptr(t.block_map), ctypes.c_int(t.nblocks), ctypes.c_float(group["lr"]),
                        ctypes.c_float(group["weight_decay"]), ctypes.c_int(int(self.use_nvlamb)), _lib.ptr(p_sq), _lib.ptr(u_sq),
                        _lib.ptr(noop_flag), ctypes.c_int(DT[pdt]), _lib.stream_ptr())
                    if rc:
                        raise RuntimeError(f"oslo_mt_lamb_stage2 failed ({rc})")
                else:
                    gnorm = math.sqrt(total_cpu + (float(total_dev) if total_dev is not None else 0.0))
                    clip = gnorm / group["max_grad_norm"] if (group["max_grad_norm"] > 0 and gnorm > group["max_grad_norm"]) else 1.0
                    for p in ps:
                        st = self.state[p]
                        pv = p.data.float()
                        g = p.grad.float() / clip
                        if not self.adam_w_mode:
                            g = g.add(pv, alpha=group["weight_decay"])
                        st["exp_avg"].mul_(b1).add_(g, alpha=beta3)
                        st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
                        upd = (st["exp_avg"] / bc1) / ((st["exp_avg_sq"] / bc2).sqrt() + group["eps"])
                        if self.adam_w_mode:
                            upd = upd.add(pv, alpha=group["weight_decay"])
                        ratio = 1.0
                        if self.use_nvlamb or group["weight_decay"] != 0:
                            pn, un = float(pv.norm()), float(upd.norm())
                            if pn > 0 and un > 0:
                                ratio = pn / un
                        p.data.add_(upd.to(p.dtype), alpha=-group["lr"] * ratio)
        return loss


class FusedMixedPrecisionLamb(FusedLamb):
    """LAMB for fp16 / bf16 training with a ``torch.amp.GradScaler``: pass the scaler to ``step`` and the kernels read
    its ``inv_scale`` and ``found_inf`` on the device."""

    @torch.no_grad()
    def step(self, closure=None, grad_scaler=None):
        inv_scale = noop = None
        if grad_scaler is not None:
            scale = grad_scaler._get_scale_async() if hasattr(grad_scaler, "_get_scale_async") else None
            if scale is not None:
                inv_scale = scale.double().reciprocal().float()
            found = getattr(grad_scaler, "_found_inf_tensor", None)
            noop = found.to(torch.int32) if found is not None else None
        return super().step(closure, inv_scale=inv_scale, noop_flag=noop)
