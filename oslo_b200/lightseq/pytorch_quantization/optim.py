"""Parameter selection helpers for quantisation-aware fine-tuning.

Parity: oslo/lightseq2/training/pytorch_quantization/optim/helper.py (``match_parameters``, ``group_parameters``,
``freeze_parameters``, ``quant_weight_inplace``).  Patterns are regular expressions matched against the start of a
parameter's qualified name (``re.match``).
"""
from __future__ import annotations

import re
from typing import Dict, Iterable, Iterator, List, Optional, Sequence

import torch
import torch.nn as nn


def match_parameters(model: nn.Module, patterns: Sequence[str]) -> Iterator[nn.Parameter]:
    """Parameters whose name matches any pattern."""
    for name, p in model.named_parameters():
        if any(re.match(pat, name) for pat in patterns):
            yield p


def group_parameters(model: nn.Module, patterns_list: Sequence[Sequence[str]], lrs: Optional[Sequence[float]] = None,
                     momentums: Optional[Sequence[float]] = None, weight_decays: Optional[Sequence[float]] = None) -> List[Dict]:
    """Optimizer parameter groups, one per pattern list, each with its own lr / momentum / weight decay when given.  A
    parameter matched by two groups is an error (an optimizer would update it twice)."""
    for opt_name, values in (("lrs", lrs), ("momentums", momentums), ("weight_decays", weight_decays)):
        if values is not None and len(values) != len(patterns_list):
            raise TypeError(f"{opt_name} needs one value per group ({len(patterns_list)})")
    groups: List[Dict] = []
    seen: Dict[int, int] = {}
    for gi, patterns in enumerate(patterns_list):
        if isinstance(patterns, str):
            patterns = [patterns]
        params = list(match_parameters(model, patterns))
        for p in params:
            if id(p) in seen:
                raise ValueError(f"a parameter is matched by groups {seen[id(p)]} and {gi}")
            seen[id(p)] = gi
        group: Dict = {"params": params}
        if lrs is not None:
            group["lr"] = lrs[gi]
        if momentums is not None:
            group["momentum"] = momentums[gi]
        if weight_decays is not None:
            group["weight_decay"] = weight_decays[gi]
        groups.append(group)
    return groups


def freeze_parameters(model: nn.Module, patterns: Sequence[str]) -> int:
    """``requires_grad = False`` on every matching parameter; returns how many were frozen."""
    n = 0
    for p in match_parameters(model, patterns):
        p.requires_grad_(False)
        n += 1
    return n


def quant_weight_inplace(model: nn.Module) -> int:
    """Overwrite each quantised layer's weight by its fake-quantised value (what the int8 engine will hold) and switch
    the weight quantiser off, so evaluation reads already-rounded weights.  Returns the number of layers rewritten."""
    n = 0
    with torch.no_grad():
        for module in model.modules():
            wq = getattr(module, "weight_quantizer", None)
            w = getattr(module, "weight", None)
            if wq is None or w is None or getattr(wq, "_disabled", False):
                continue
            if not wq.fake_quant:
                raise ValueError("in-place weight quantisation needs fake_quant descriptors")
            w.copy_(wq(w))
            wq.disable()
            n += 1
    return n


__all__ = ["match_parameters", "group_parameters", "freeze_parameters", "quant_weight_inplace"]
