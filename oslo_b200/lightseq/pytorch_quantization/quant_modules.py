"""Swap float layers for their quantised versions: globally (newly built models) or in an existing model.

Parity: oslo/lightseq2/training/pytorch_quantization/quant_modules.py (``initialize`` / ``deactivate`` patch the classes in
``torch.nn`` so that a model constructed afterwards is quantised).  :func:`replace_with_quant` is the in-place variant for a
model that already exists (and already holds trained weights): each supported layer becomes its quantised subclass with
the same parameters, no copy.
"""
from __future__ import annotations

import contextlib
from typing import Dict, Iterable, List, Optional, Tuple

import torch.nn as tnn

from . import nn as qnn

_DEFAULT_MAP: Tuple[Tuple[str, type], ...] = (
    ("Linear", qnn.QuantLinear),
    ("Conv1d", qnn.QuantConv1d), ("Conv2d", qnn.QuantConv2d), ("Conv3d", qnn.QuantConv3d),
    ("ConvTranspose1d", qnn.QuantConvTranspose1d), ("ConvTranspose2d", qnn.QuantConvTranspose2d),
    ("ConvTranspose3d", qnn.QuantConvTranspose3d),
    ("MaxPool1d", qnn.QuantMaxPool1d), ("MaxPool2d", qnn.QuantMaxPool2d), ("MaxPool3d", qnn.QuantMaxPool3d),
    ("AvgPool1d", qnn.QuantAvgPool1d), ("AvgPool2d", qnn.QuantAvgPool2d), ("AvgPool3d", qnn.QuantAvgPool3d),
    ("AdaptiveAvgPool1d", qnn.QuantAdaptiveAvgPool1d), ("AdaptiveAvgPool2d", qnn.QuantAdaptiveAvgPool2d),
    ("AdaptiveAvgPool3d", qnn.QuantAdaptiveAvgPool3d),
    ("InstanceNorm1d", qnn.QuantInstanceNorm1d), ("InstanceNorm2d", qnn.QuantInstanceNorm2d),
    ("InstanceNorm3d", qnn.QuantInstanceNorm3d),
)


class QuantModuleReplacementHelper:
    """Keeps the original classes so that :meth:`restore_float_modules` puts back exactly what was replaced."""

    def __init__(self):
        self._originals: List[Tuple[object, str, type]] = []
        self._plan: List[Tuple[object, str, type]] = []

    def prepare_state(self, float_module_list: Optional[Iterable[str]] = None, custom_map: Optional[Iterable[Tuple[object, str, type]]] = None):
        """``float_module_list``: names to leave as float.  ``custom_map``: extra ``(python module, class name, quantised
        class)`` triples (they replace a default entry of the same name in ``torch.nn``)."""
        skip = set(float_module_list or ())
        plan: Dict[Tuple[int, str], Tuple[object, str, type]] = {}
        for name, qcls in _DEFAULT_MAP:
            if name not in skip:
                plan[(id(tnn), name)] = (tnn, name, qcls)
        for mod, name, qcls in custom_map or ():
            plan[(id(mod), name)] = (mod, name, qcls)
        self._plan = list(plan.values())

    def apply_quant_modules(self):
        for mod, name, qcls in self._plan:
            self._originals.append((mod, name, getattr(mod, name)))
            setattr(mod, name, qcls)

    def restore_float_modules(self):
        for mod, name, orig in reversed(self._originals):
            setattr(mod, name, orig)
        self._originals = []


_helper = QuantModuleReplacementHelper()


def initialize(float_module_list: Optional[Iterable[str]] = None, custom_quant_modules=None) -> None:
    """From now on ``torch.nn.Linear`` etc. construct quantised layers.  Call :func:`deactivate` to undo."""
    if _helper._originals:
        raise RuntimeError("already initialised; call deactivate() first")
    _helper.prepare_state(float_module_list, custom_quant_modules)
    _helper.apply_quant_modules()


def deactivate() -> None:
    _helper.restore_float_modules()


@contextlib.contextmanager
def quantized_construction(float_module_list=None, custom_quant_modules=None):
    """Context-manager form of initialize / deactivate."""
    initialize(float_module_list, custom_quant_modules)
    try:
        yield
    finally:
        deactivate()



def replace_with_quant(model: tnn.Module, skip: Iterable[str] = (), quant_desc_input=None, quant_desc_weight=None) -> int:
    """Turn every supported float layer of ``model`` into its quantised subclass in place (parameters shared, module
    identity kept, so optimizers and hooks stay valid).  ``skip``: qualified-name prefixes to leave alone (typically the
    output head).  Returns the number of layers converted."""
    skip = tuple(skip)
    table = {getattr(tnn, name): qcls for name, qcls in _DEFAULT_MAP if not _helper._originals}
    if _helper._originals:  # torch.nn is patched right now: key the table by the saved float classes
        table = {orig: getattr(mod, name) for mod, name, orig in _helper._originals if mod is tnn}
    count = 0
    for name, module in model.named_modules():
        if any(name == s or name.startswith(s + ".") for s in skip):
            continue
        qcls = table.get(type(module))
        if qcls is None:
            continue
        module.__class__ = qcls
        if hasattr(qcls, "default_quant_desc_weight"):
            module.init_quantizer(quant_desc_input, quant_desc_weight)
        else:
            module.init_quantizer(quant_desc_input)
        for q in (getattr(module, "input_quantizer", None), getattr(module, "weight_quantizer", None)):
            if q is not None and hasattr(module, "weight") and module.weight is not None:
                q.to(module.weight.device)
        count += 1
    return count


__all__ = ["QuantModuleReplacementHelper", "initialize", "deactivate", "quantized_construction", "replace_with_quant"]
