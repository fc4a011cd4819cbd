"""Validated nested configuration (dict or JSON file) -> ``ParallelContext`` + model wrappers.

Schema (unknown keys are rejected, values are type / enum checked), as the reference's ``SUPPORTED_FEATURES``
(oslo/transformers/oslo_init.py:47-126):

    backend:                 {name: nccl|gloo, host, port}
    mixed_precision:         {enable: bool, dtype: bf16|fp16}
    activation_checkpointing:{partitioned: bool, contiguous: bool, cpu: bool}
    sequence_parallelism:    {parallel_size: int}
    data_parallelism:        {parallel_size: int, zero_stage: 0..3, params: {cpu_offload: bool, ...}}
    tensor_parallelism:      {parallel_size: int, parallel_mode: 1d|2d|2.5d|3d, sequence_parallel: bool,
                              params: {parallel_depth_2.5d: int}}
    pipeline_parallelism:    {parallel_size: int, params: {memory_computation_balance: float, num_micro_batches: int}}
    expert_parallelism:      {parallel_size: int, params: {top_k, capacity_factor_train, num_dec_experts, ...}}

Unlike the reference, the 2.5-D depth is read from ``params`` (it reads a misspelt key and ignores it,
oslo_init.py:386-392) and the expert wrapper is actually added (:438-445).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional, Tuple

from oslo_b200.distributed import ParallelContext, ParallelMode

_bool = lambda v: isinstance(v, bool)
_int = lambda v: isinstance(v, int) and not isinstance(v, bool)
_pos = lambda v: _int(v) and v >= 1
_num = lambda v: isinstance(v, (int, float)) and not isinstance(v, bool)
_str = lambda v: isinstance(v, str)
_any = lambda v: True

SUPPORTED_FEATURES: Dict[str, Any] = {
    "backend": {"name": lambda v: v in ("nccl", "gloo"), "host": _str, "port": lambda v: _int(v) or _str(v)},
    "mixed_precision": {"enable": _bool, "dtype": lambda v: v in ("bf16", "fp16")},
    "activation_checkpointing": {"partitioned": _bool, "contiguous": _bool, "cpu": _bool},
    "sequence_parallelism": {"parallel_size": _pos},
    "data_parallelism": {"parallel_size": _pos, "zero_stage": lambda v: v in (0, 1, 2, 3),
                         "params": {"cpu_offload": _bool, "overlap_communication": _bool, "clip_grad_norm": _num,
                                    "reduce_bucket_size": _pos}},
    "tensor_parallelism": {"parallel_size": _pos, "parallel_mode": lambda v: v in ("1d", "2d", "2.5d", "3d"),
                           "sequence_parallel": _bool, "params": {"parallel_depth_2.5d": _pos}},
    "pipeline_parallelism": {"parallel_size": _pos,
                             "params": {"memory_computation_balance": _num, "num_micro_batches": _pos}},
    "expert_parallelism": {"parallel_size": _pos,
                           "params": {"top_k": lambda v: v in (1, 2), "capacity_factor_train": _num,
                                      "capacity_factor_eval": _num, "min_capacity": _int, "use_rts": _bool,
                                      "drop_tokens": _bool, "num_enc_experts": _any, "num_dec_experts": _any,
                                      "aux_loss_coef": _num, "noisy_policy": lambda v: v in (None, "Jitter", "RSample")}},
}


def _config_check(schema: dict, cfg: dict, path: str = ""):
    for key, value in cfg.items():
        where = f"{path}.{key}" if path else key
        if key not in schema:
            raise KeyError(f"unknown configuration key '{where}'; allowed: {sorted(schema)}")
        rule = schema[key]
        if isinstance(rule, dict):
            if not isinstance(value, dict):
                raise TypeError(f"'{where}' must be a mapping")
            _config_check(rule, value, where)
        elif not rule(value):
            raise ValueError(f"invalid value {value!r} for '{where}'")


class OsloTrainerConfig:
    def __init__(self, config_path_or_dict):
        if isinstance(config_path_or_dict, dict):
            cfg = config_path_or_dict
        elif isinstance(config_path_or_dict, (str, os.PathLike)):
            with open(config_path_or_dict) as f:
                cfg = json.load(f)
        else:
            raise TypeError("oslo config must be a dict or the path of a JSON file")
        _config_check(SUPPORTED_FEATURES, cfg)
        self.raw = cfg
        for key in SUPPORTED_FEATURES:
            setattr(self, key, cfg.get(key))

    def size(self, feature: str) -> int:
        sec = getattr(self, feature)
        return int(sec.get("parallel_size", 1)) if sec else 1

    def __repr__(self):
        return f"OsloTrainerConfig({json.dumps(self.raw, indent=1)})"


_MODES = {"1d": ParallelMode.TENSOR_1D, "2d": ParallelMode.TENSOR_2D, "2.5d": ParallelMode.TENSOR_2P5D,
          "3d": ParallelMode.TENSOR_3D}


def init_oslo_features(cfg: OsloTrainerConfig) -> Tuple[ParallelContext, List[tuple]]:
    """Build the ``ParallelContext`` from the launcher's environment and the list of wrapper recipes
    ``[(wrapper_class, kwargs), ...]`` to apply to a model (see :func:`apply_wrappers`)."""
    tp = cfg.tensor_parallelism or {}
    backend = cfg.backend or {}
    kwargs = dict(
        data_parallel_size=cfg.size("data_parallelism"),
        sequence_parallel_size=cfg.size("sequence_parallelism"),
        expert_parallel_size=cfg.size("expert_parallelism"),
        pipeline_parallel_size=cfg.size("pipeline_parallelism"),
        tensor_parallel_size=cfg.size("tensor_parallelism"),
        tensor_parallel_mode=_MODES[tp.get("parallel_mode", "1d")],
        tensor_parallel_depth=(tp.get("params") or {}).get("parallel_depth_2.5d"),
        backend=backend.get("name", "nccl"),
    )
    env = os.environ
    if "SLURM_PROCID" in env and "RANK" not in env:
        pc = ParallelContext.from_slurm(backend.get("host", "127.0.0.1"), int(backend.get("port", 29500)), **kwargs)
    elif "OMPI_COMM_WORLD_RANK" in env and "RANK" not in env:
        pc = ParallelContext.from_openmpi(backend.get("host", "127.0.0.1"), int(backend.get("port", 29500)), **kwargs)
    else:
        pc = ParallelContext.from_torch(**kwargs)

    from oslo_b200.parallel import ExpertParallel, PipelineParallel, TensorParallel

    recipes: List[tuple] = []
    if cfg.size("tensor_parallelism") > 1:
        recipes.append((TensorParallel, dict(sequence_parallel=bool(tp.get("sequence_parallel", False)))))
    if cfg.expert_parallelism:
        recipes.append((ExpertParallel, dict(cfg.expert_parallelism.get("params") or {})))
    if cfg.size("pipeline_parallelism") > 1:
        recipes.append((PipelineParallel, dict((cfg.pipeline_parallelism.get("params") or {}))))
    return pc, recipes


def apply_wrappers(model, pc: ParallelContext, recipes: List[tuple]):
    """Register every wrapper on ``model`` (``oslo_b200.ready`` then applies them in priority order) and return the
    outermost one, which is what the training loop calls."""
    wrapped = model
    for cls, kw in recipes:
        wrapped = cls(model, pc, **kw)
    return wrapped
