"""Adam / AdamW and Adagrad whose parameters and state live in host memory (``csrc/cpu/cpu_optim.cpp``).

The update runs on the CPU (AVX-512 / AVX2 + OpenMP).  With ``param_copies`` (a dict ``cpu_param -> device tensor``)
each step also produces a 16-bit copy of the new parameters in pinned memory in the same pass and ships it to the
device asynchronously, so only half the bytes cross PCIe.
Parity: oslo/torch/optim/cpu_adam.py:10-208, cpu_adagrad.py.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch

from oslo_b200.ops import _lib

_LOWP = {torch.float16: 1, torch.bfloat16: 2}


def _fptr(t):
    return ctypes.c_void_p(t.data_ptr())


class CPUAdam(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, bias_correction=True, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                 amsgrad=False, adamw_mode=True, param_copies: Optional[Dict[torch.Tensor, torch.Tensor]] = None):
        if amsgrad:
            raise RuntimeError("CPUAdam does not support the AMSGrad variant")
        super().__init__(params, dict(lr=lr, bias_correction=bias_correction, betas=betas, eps=eps, weight_decay=weight_decay))
        self.adamw_mode = 1 if adamw_mode else 0
        self.param_copies = param_copies or {}
        self._staging: Dict[int, torch.Tensor] = {}
        self.lib = _lib.cpu_lib()
        self.simd_level = self.lib.oslo_cpu_simd_level()

    @torch.no_grad()
    def step(self, closure=None, grad_scale: float = 1.0):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            group["step"] = group.get("step", 0) + 1
            b1, b2 = group["betas"]
            t = group["step"]
            bc1 = 1 - b1**t if group["bias_correction"] else 1.0
            bc2 = 1 - b2**t if group["bias_correction"] else 1.0
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.device.type != "cpu" or p.dtype != torch.float32:
                    raise RuntimeError("CPUAdam needs fp32 parameters in host memory")
                st = self.state[p]
                if not st:
                    st["exp_avg"] = torch.zeros_like(p)
                    st["exp_avg_sq"] = torch.zeros_like(p)
                g = p.grad.float().contiguous()
                dev = self.param_copies.get(p)
                lowp, kind = None, 0
                if dev is not None and dev.dtype in _LOWP:
                    lowp = self._staging.get(id(p))
                    if lowp is None:
                        lowp = torch.empty(p.numel(), dtype=dev.dtype)
                        if torch.cuda.is_available():
                            lowp = lowp.pin_memory()
                        self._staging[id(p)] = lowp
                    kind = _LOWP[dev.dtype]
                self.lib.oslo_cpu_adam_step(
                    _fptr(p.data), _fptr(g), _fptr(st["exp_avg"]), _fptr(st["exp_avg_sq"]), ctypes.c_longlong(p.numel()),
                    ctypes.c_float(group["lr"]), ctypes.c_float(b1), ctypes.c_float(b2), ctypes.c_float(group["eps"]),
                    ctypes.c_float(group["weight_decay"]), ctypes.c_float(bc1), ctypes.c_float(bc2), ctypes.c_float(grad_scale),
                    ctypes.c_int(self.adamw_mode), _fptr(lowp) if lowp is not None else None, ctypes.c_int(kind))
                if dev is not None:
                    src = lowp.view(p.shape) if lowp is not None else p.data
                    dev.copy_(src, non_blocking=True)
        return loss


class CPUAdagrad(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-2, eps=1e-10, weight_decay=0.0, param_copies=None):
        super().__init__(params, dict(lr=lr, eps=eps, weight_decay=weight_decay))
        self.param_copies = param_copies or {}
        self.lib = _lib.cpu_lib()

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["sum"] = torch.zeros_like(p)
                g = p.grad.float().contiguous()
                self.lib.oslo_cpu_adagrad_step(_fptr(p.data), _fptr(g), _fptr(st["sum"]), ctypes.c_longlong(p.numel()),
                                               ctypes.c_float(group["lr"]), ctypes.c_float(group["eps"]),
                                               ctypes.c_float(group["weight_decay"]), None, ctypes.c_int(0))
                dev = self.param_copies.get(p)
                if dev is not None:
                    dev.copy_(p.data.to(dev.dtype), non_blocking=True)
        return loss
