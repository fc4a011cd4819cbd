"""Declarative description of how a model's modules are tensor-parallelised.

A mapping is a list of ``Column(...)``, ``Row(...)``, ``Update(...)``, ``Head(...)``, ``Other(...)`` entries
whose names are matched against dotted module / attribute names (whole dotted components, so ``"dense"``
matches ``attention.dense`` but not ``dense_h_to_4h``).

Parity: oslo/torch/nn/parallel/tensor_parallel/mapping.py:4-180.
"""
from __future__ import annotations

import copy
from typing import Dict, List, Optional


class TensorParallelInfo:
    def __init__(self, *name, combined_qkv: bool = False, reversed: bool = False, gather_output: bool = False):
        self.name = name
        self.combined_qkv = combined_qkv
        self.reversed = reversed
        self.gather_output = gather_output

    def __repr__(self):
        return f"{self.__class__.__qualname__}({self.name})"


class Column(TensorParallelInfo):
    pass


class Row(TensorParallelInfo):
    pass


class Update(TensorParallelInfo):
    pass


class Head(TensorParallelInfo):
    pass


class Other(TensorParallelInfo):
    pass


def _name_matches(pattern: str, full_name: str) -> bool:
    """``pattern`` (possibly dotted) must equal a run of whole dotted components of ``full_name``."""
    pat = pattern.split(".")
    parts = full_name.split(".")
    n = len(pat)
    return any(parts[i : i + n] == pat for i in range(len(parts) - n + 1))


class TensorParallelMapping:
    __MAPPING__: Dict[str, List[TensorParallelInfo]] = {}

    def __init__(self, tp_mapping: Optional[dict] = None):
        table = dict(self.__MAPPING__)
        if isinstance(tp_mapping, dict):
            table.update(tp_mapping)
        elif tp_mapping is not None:
            raise ValueError("tp_mapping must be None or a dict")
        self._table = {}
        for key, entries in table.items():
            flat = []
            for e in entries:
                for n in e.name:
                    c = copy.copy(e)
                    c.name = n
                    flat.append(c)
            self._table[key] = flat

    def get_mapping(self, model) -> Optional[List[TensorParallelInfo]]:
        """Entries of the longest table key that prefixes any class name in the model's MRO."""
        best = None
        for cls in type(model).__mro__:
            for key, entries in self._table.items():
                k = key if isinstance(key, str) else key.__name__
                if cls.__name__.startswith(k) and (best is None or len(k) > best[0]):
                    best = (len(k), entries)
            if best is not None:
                break
        return best[1] if best else None

    def search(self, model, param_name: str) -> Optional[TensorParallelInfo]:
        mapping = self.get_mapping(model)
        if mapping is None:
            raise ValueError(f"{type(model).__name__} has no tensor-parallel mapping; pass one explicitly")
        name = param_name
        for suffix in (".weight", ".bias"):
            if name.endswith(suffix):
                name = name[: -len(suffix)]
        hits = [e for e in mapping if _name_matches(e.name, name)]
        if not hits:
            return None
        return max(hits, key=lambda e: len(e.name))

    def _is(self, model, name, kind):
        e = self.search(model, name)
        return e is not None and isinstance(e, kind)

    def is_column_parallel(self, model, name):
        return self._is(model, name, Column)

    def is_row_parallel(self, model, name):
        return self._is(model, name, Row)

    def is_head(self, model, name):
        return self._is(model, name, Head)

    def is_other(self, model, name):
        return self._is(model, name, Other)

    def update_attrs(self, model) -> List[str]:
        mapping = self.get_mapping(model) or []
        return [e.name for e in mapping if isinstance(e, Update)]

    def is_combined_qkv_param(self, model, name):
        e = self.search(model, name)
        return bool(e is not None and e.combined_qkv)

    def is_reversed(self, model, name):
        e = self.search(model, name)
        return bool(e is not None and e.reversed)

    def is_gather_output(self, model, name):
        e = self.search(model, name)
        return bool(e is not None and e.gather_output)

    @staticmethod
    def get_combined_qkv_degree(weight) -> int:
        """3 for fused QKV, 2 for fused KV: ratio of the long to the short side of the weight."""
        return max(weight.shape) // min(weight.shape)
