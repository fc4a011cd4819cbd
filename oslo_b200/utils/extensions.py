"""``ready`` plus the sharded / merged checkpoint functions it attaches to a model.

* ``save_pretrained(dir)`` writes ``pytorch_model_tp_{t}_pp_{p}_ep_{e}.bin`` (this rank's shards, unmodified
  state-dict keys) from data-parallel rank 0 only, plus ``config.json``.
* ``save_pretrained(dir, merge_checkpoints=True)`` merges all shards (all-gathers driven by each parameter's
  shard spec) and rank 0 writes one ``pytorch_model.bin`` identical to the unsharded model's.
* ``from_parallelized(dir)`` loads this rank's file; all ``tp x pp x ep`` files must exist.

Unlike the reference (oslo/torch/utils/extensions.py:36-121), merging does not build a second full-size model
on every rank: tensors are merged one by one from the live shards.

Parity: oslo/torch/utils/extensions.py:36-275.
"""
from __future__ import annotations

import copy
import json
import os
import types
from typing import Callable, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from oslo_b200.distributed import ParallelMode
from oslo_b200.parallel.utils import parallelize, unwrap_parallel

PARALLELIZED_WEIGHTS_NAME = "pytorch_model_tp_{tp}_pp_{pp}_ep_{ep}.bin"
WEIGHTS_NAME = "pytorch_model.bin"


def _ranks(pc):
    def r(mode):
        return pc.get_local_rank(mode) if pc.is_initialized(mode) else 0

    return r(ParallelMode.TENSOR), r(ParallelMode.PIPELINE), r(ParallelMode.EXPERT)


def _save_config(base, save_directory):
    cfg = getattr(base, "config", None)
    if cfg is None:
        return
    cfg = copy.deepcopy(cfg)
    try:
        dtype = next(base.parameters()).dtype
        cfg.torch_dtype = str(dtype).split(".")[1]
    except StopIteration:
        pass
    cfg.architectures = [base.__class__.__name__]
    if hasattr(base, "orig_vocab_size") and hasattr(cfg, "vocab_size"):
        cfg.vocab_size = base.orig_vocab_size
    if hasattr(cfg, "save_pretrained"):
        try:
            cfg.save_pretrained(save_directory)
            return
        except Exception:
            pass
    with open(os.path.join(save_directory, "config.json"), "w") as f:
        json.dump(cfg.to_dict() if hasattr(cfg, "to_dict") else cfg.__dict__, f, indent=2, default=str)


def _merged_state_dict(model, pc):
    """Full (unsharded) state dict assembled from live shards; collective over TP / PP / EP groups."""
    from oslo_b200.parallel.tensor_parallel._sharding import merge

    base = unwrap_parallel(model)
    out = {}
    cache = {}
    for key, p in base.state_dict(keep_vars=True).items():
        spec = getattr(p, "oslo_shard", None)
        if getattr(p, "oslo_pipeline_released", False):
            # another pipeline stage owns this tensor (every rank of this tensor-parallel group released it, so skipping
            # the merge keeps the collective order identical inside the group); the pipeline hook below fills it in
            out[key] = p.detach().cpu()
        elif spec is not None:
            if id(p) not in cache:
                cache[id(p)] = merge(p.data, spec, pc).cpu()
            out[key] = cache[id(p)]
        else:
            out[key] = p.detach().cpu()
    for wrapper in getattr(base, "oslo_wrappers", {}).values():
        hook = getattr(wrapper, "merge_state_dict_hook", None)
        if hook is not None:
            out = hook(out)
    return out


def save_pretrained(self, save_directory: str, save_config: bool = True, state_dict: Optional[dict] = None,
                    save_function: Callable = torch.save, merge_checkpoints: bool = False, **kwargs):
    pc = self.parallel_context
    base = unwrap_parallel(self)
    os.makedirs(save_directory, exist_ok=True)
    dp_rank = pc.get_local_rank(ParallelMode.DATA) if pc.is_initialized(ParallelMode.DATA) else 0
    if merge_checkpoints:
        merged = _merged_state_dict(self, pc)
        if pc.get_global_rank() == 0:
            if save_config:
                _save_config(base, save_directory)
            save_function(merged, os.path.join(save_directory, WEIGHTS_NAME))
        if dist.is_initialized():
            dist.barrier()
        return
    if dp_rank == 0:
        tp, pp, ep = _ranks(pc)
        if save_config and tp == 0 and pp == 0 and ep == 0:
            _save_config(base, save_directory)
        sd = state_dict if state_dict is not None else base.state_dict()
        sd = {k: v.detach().cpu() for k, v in sd.items()}
        save_function(sd, os.path.join(save_directory, PARALLELIZED_WEIGHTS_NAME.format(tp=tp, pp=pp, ep=ep)))
    if dist.is_initialized():
        dist.barrier()


def from_parallelized(self, path: str, strict: bool = False):
    """Load this rank's shard file written by ``save_pretrained``; every rank's file must be present."""
    pc = self.parallel_context
    base = unwrap_parallel(self)
    if not os.path.isdir(path):
        raise NotADirectoryError(f"{path} is not a directory")
    tp_size = pc.get_world_size(ParallelMode.TENSOR) if pc.is_initialized(ParallelMode.TENSOR) else 1
    pp_size = pc.get_world_size(ParallelMode.PIPELINE) if pc.is_initialized(ParallelMode.PIPELINE) else 1
    ep_size = pc.get_world_size(ParallelMode.EXPERT) if pc.is_initialized(ParallelMode.EXPERT) else 1
    missing = [
        PARALLELIZED_WEIGHTS_NAME.format(tp=t, pp=p, ep=e)
        for t in range(tp_size) for p in range(pp_size) for e in range(ep_size)
        if not os.path.isfile(os.path.join(path, PARALLELIZED_WEIGHTS_NAME.format(tp=t, pp=p, ep=e)))
    ]
    if missing:
        raise FileNotFoundError(f"all {tp_size * pp_size * ep_size} shard files are needed; missing: {missing}")
    tp, pp, ep = _ranks(pc)
    sd = torch.load(os.path.join(path, PARALLELIZED_WEIGHTS_NAME.format(tp=tp, pp=pp, ep=ep)), map_location="cpu")
    result = base.load_state_dict(sd, strict=strict)
    if hasattr(base, "tie_weights"):
        pass  # tied parameters are shared objects; loading one key fills both
    return result


def _blocked_resize(self, *args, **kwargs):
    raise RuntimeError("resize_token_embeddings() is not available after oslo_b200.ready(): resize before wrapping")


def ready(model: nn.Module, parallel_context):
    """Apply every registered wrapper, move the model to this rank's device and attach the checkpoint methods."""
    parallelize(model, parallel_context)
    base = unwrap_parallel(model)
    for obj in {id(model): model, id(base): base}.values():
        obj.parallel_context = parallel_context
        obj.save_pretrained = types.MethodType(save_pretrained, obj)
        obj.from_parallelized = types.MethodType(from_parallelized, obj)
        if hasattr(obj, "resize_token_embeddings") or obj is base:
            obj.resize_token_embeddings = types.MethodType(_blocked_resize, obj)
    return model
