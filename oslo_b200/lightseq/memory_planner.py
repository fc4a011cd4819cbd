"""Static activation-memory planning (``csrc/cpu/memory_planner.cpp``) and a tracer that plans a module's forward.

``plan(sizes, first_use, last_use)`` returns ``(offsets, total)``.  ``ActivationPlan.trace(module, *inputs)`` runs one
dry forward pass with hooks, records when every leaf module's output is produced and last consumed, and plans one
shared arena for them; ``arena_bytes`` versus ``naive_bytes`` tells how much a static executor would save.

Counterpart of lightseq2's lsflow ``MemoryManager`` / ``Context`` dry-run
(oslo/lightseq2/csrc/lsflow/manager.cpp:29-232, context.cpp:5-193).
"""
from __future__ import annotations

import ctypes
from typing import List, Sequence, Tuple

import torch
import torch.nn as nn

from oslo_b200.ops import _lib


def plan(sizes: Sequence[int], first_use: Sequence[int], last_use: Sequence[int], alignment: int = 256) -> Tuple[List[int], int]:
    n = len(sizes)
    arr = lambda v: (ctypes.c_longlong * n)(*[int(x) for x in v])
    offsets = (ctypes.c_longlong * n)()
    lib = _lib.cpu_lib()
    lib.oslo_plan_memory.restype = ctypes.c_longlong
    total = lib.oslo_plan_memory(arr(sizes), arr(first_use), arr(last_use), ctypes.c_int(n), ctypes.c_longlong(alignment), offsets)
    if total < 0:
        raise ValueError("invalid sizes / lifetimes")
    return list(offsets), int(total)


def check(sizes, first_use, last_use, offsets) -> bool:
    n = len(sizes)
    arr = lambda v: (ctypes.c_longlong * n)(*[int(x) for x in v])
    return _lib.cpu_lib().oslo_check_memory_plan(arr(sizes), arr(first_use), arr(last_use), arr(offsets), ctypes.c_int(n)) == 0


class ActivationPlan:
    def __init__(self, names, sizes, first, last, offsets, total):
        self.names, self.sizes, self.first, self.last, self.offsets = names, sizes, first, last, offsets
        self.arena_bytes = total
        self.naive_bytes = sum(sizes)

    @classmethod
    def trace(cls, module: nn.Module, *args, alignment: int = 256, **kwargs) -> "ActivationPlan":
        names, sizes, first, last = [], [], [], []
        produced = {}  # data_ptr -> index
        clock = [0]
        hooks = []

        def pre(mod, inputs):
            clock[0] += 1
            for t in inputs:
                if torch.is_tensor(t) and t.data_ptr() in produced:
                    last[produced[t.data_ptr()]] = clock[0]

        def post(mod, inputs, out):
            outs = out if isinstance(out, (tuple, list)) else (out,)
            for t in outs:
                if torch.is_tensor(t) and t.data_ptr() not in produced:
                    produced[t.data_ptr()] = len(sizes)
                    names.append(names_of.get(id(mod), mod.__class__.__name__))
                    sizes.append(t.numel() * t.element_size())
                    first.append(clock[0])
                    last.append(clock[0])

        names_of = {id(m): n for n, m in module.named_modules()}
        for m in module.modules():
            if len(list(m.children())) == 0:
                hooks.append(m.register_forward_pre_hook(pre))
                hooks.append(m.register_forward_hook(post))
        with torch.no_grad():
            module(*args, **kwargs)
        for h in hooks:
            h.remove()
        offsets, total = plan(sizes, first, last, alignment)
        assert check([(s + alignment - 1) // alignment * alignment for s in sizes], first, last, offsets)
        return cls(names, sizes, first, last, offsets, total)
