"""Adam / AdamW with one kernel launch per (param group, dtype) and fp32 math.

On CUDA the whole group is updated by ``oslo_mt_adam`` through a device-resident
tensor table (see :mod:`oslo_b200.ops.multi_tensor`); bf16 / fp16 parameters can keep
fp32 master copies (``master_weights=True``).  On CPU tensors the same update is
computed with torch ops, bit-compatible with ``torch.optim.AdamW`` for fp32.

Parity: oslo/torch/optim/fused_adam.py:16-184 (which rejects bf16, :150-151).
"""
from __future__ import annotations

import ctypes
import math
from typing import Dict, List

import torch

from oslo_b200.ops import _lib
from oslo_b200.ops.multi_tensor import TensorTable

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


class FusedAdam(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, bias_correction=True, betas=(0.9, 0.999), eps=1e-8, adam_w_mode=True,
                 weight_decay=0.0, amsgrad=False, set_grad_none=True, master_weights=False, capturable=False):
        if amsgrad:
            raise RuntimeError("FusedAdam does not support the AMSGrad variant")
        defaults = dict(lr=lr, bias_correction=bias_correction, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.adam_w_mode = 1 if adam_w_mode else 0
        self.set_grad_none = set_grad_none
        self.master_weights = master_weights
        #: keep the step count on the device and compute bias corrections in the kernel, so ``step()`` can be captured
        #: in a CUDA graph and replayed
        self.capturable = capturable
        self._step_dev = {}
        self._tables: Dict[tuple, TensorTable] = {}

    def zero_grad(self, set_to_none: bool = None):
        if set_to_none is None:
            set_to_none = self.set_grad_none
        super().zero_grad(set_to_none=set_to_none)

    def _init_state(self, p):
        st = self.state[p]
        if len(st) == 0:
            st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
            st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
            if self.master_weights and p.dtype != torch.float32:
                st["master"] = p.detach().float().clone()
        return st

    @torch.no_grad()
    def step(self, closure=None, grad_scale: float = 1.0, inv_scale=None, noop_flag=None):
        loss = closure() if closure is not None else None
        for gi, group in enumerate(self.param_groups):
            group["step"] = group.get("step", 0) + 1
            step = group["step"]
            b1, b2 = group["betas"]
            bc1 = 1 - b1**step if group["bias_correction"] else 1.0
            bc2 = 1 - b2**step if group["bias_correction"] else 1.0
            if self.capturable:
                first = next((p for p in group["params"] if p.is_cuda), None)
                if first is not None:
                    if gi not in self._step_dev:
                        self._step_dev[gi] = torch.zeros(1, dtype=torch.int32, device=first.device)
                    self._step_dev[gi].add_(1)
            buckets: Dict[tuple, List[torch.Tensor]] = {}
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("FusedAdam does not support sparse gradients")
                self._init_state(p)
                key = (p.is_cuda, p.dtype, p.grad.dtype)
                buckets.setdefault(key, []).append(p)
            for (is_cuda, pdt, gdt), ps in buckets.items():
                if is_cuda and _lib.has_cuda_kernels() and pdt in _DT and gdt in _DT:
                    self._step_cuda(gi, ps, group, bc1, bc2, pdt, gdt, grad_scale, inv_scale, noop_flag)
                else:
                    self._step_torch(ps, group, bc1, bc2, grad_scale)
        return loss

    def _step_cuda(self, gi, ps, group, bc1, bc2, pdt, gdt, grad_scale, inv_scale, noop_flag):
        grads = [p.grad if p.grad.is_contiguous() else p.grad.contiguous() for p in ps]
        datas = [p.data for p in ps]
        m = [self.state[p]["exp_avg"] for p in ps]
        v = [self.state[p]["exp_avg_sq"] for p in ps]
        master = [self.state[p]["master"] for p in ps] if "master" in self.state[ps[0]] else None
        cols = [datas, grads, m, v, master]
        key = (gi, pdt, gdt)
        table = self._tables.get(key)
        if table is None or table.n != len(ps):
            table = self._tables[key] = TensorTable(cols)
        else:
            table.update(cols)
        b1, b2 = group["betas"]
        rc = _lib.cuda_lib().oslo_mt_adam(
            _lib.ptr(table.table), _lib.ptr(table.block_map), ctypes.c_int(table.nblocks),
            ctypes.c_float(group["lr"]), ctypes.c_float(b1), ctypes.c_float(b2), ctypes.c_float(group["eps"]),
            ctypes.c_float(group["weight_decay"]), ctypes.c_float(bc1), ctypes.c_float(bc2),
            ctypes.c_float(grad_scale), ctypes.c_int(self.adam_w_mode), _lib.ptr(inv_scale), _lib.ptr(noop_flag),
            ctypes.c_int(_DT[pdt]), ctypes.c_int(_DT[gdt]), _lib.stream_ptr(),
            _lib.ptr(self._step_dev.get(gi)) if self.capturable and group["bias_correction"] else None)
        if rc:
            raise RuntimeError(f"oslo_mt_adam failed ({rc})")

    def _step_torch(self, ps, group, bc1, bc2, grad_scale):
        b1, b2 = group["betas"]
        lr, eps, wd = group["lr"], group["eps"], group["weight_decay"]
        for p in ps:
            st = self.state[p]
            g = p.grad.float() * grad_scale if (grad_scale != 1.0 or p.grad.dtype != torch.float32) else p.grad
            pv = st.get("master", p.data if p.dtype == torch.float32 else p.data.float())
            if self.adam_w_mode:
                pv.mul_(1 - lr * wd)
            elif wd != 0:
                g = g.add(pv, alpha=wd)
            st["exp_avg"].lerp_(g, 1 - b1)
            st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
            denom = (st["exp_avg_sq"].sqrt() / math.sqrt(bc2)).add_(eps)
            pv.addcdiv_(st["exp_avg"], denom, value=-lr / bc1)
            if pv is not p.data:
                p.data.copy_(pv)
