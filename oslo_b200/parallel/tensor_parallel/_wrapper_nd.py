"""Sharding plans for 2D / 2.5D / 3D tensor parallelism (the 1D plan lives in ``tensor_parallel.py``).

For each mode a small table says how every kind of parameter is split — as an ordered list of
``Split(mode, dim, parts)`` — and which parallel layer replaces the module.  Layouts follow the reference so
per-rank checkpoint files interchange (oslo/torch/nn/parallel/tensor_parallel/_2d/_wrapper.py:235-425,
_2p5d/_wrapper.py:241-262, _3d/_wrapper.py:252-300).

Labels are NOT scattered with the other inputs for the vocab-parallel losses (those split the targets
themselves, as the reference's loss modules do); for the 3D plain loss they are.
"""
from __future__ import annotations

import torch
import torch.nn as nn

import oslo_b200.nn as onn
from oslo_b200.distributed import ParallelMode, comm
from oslo_b200.transformers.constants import BATCH_DIMENSIONS_TP

from ._sharding import ShardSpec, Split

M = ParallelMode


def batch_modes(pc):
    mode = pc.tensor_parallel_mode
    if mode == M.TENSOR_2D:
        return [M.TENSOR_2D_COL]
    if mode == M.TENSOR_2P5D:
        return [M.TENSOR_2P5D_DEP, M.TENSOR_2P5D_COL]
    if mode == M.TENSOR_3D:
        return [M.TENSOR_3D_WEIGHT, M.TENSOR_3D_INPUT]
    return []


def scatter_batch_inputs(module, args, kwargs, pc):
    if args:
        raise TypeError("N-D tensor-parallel models take keyword arguments only: model(input_ids=..., labels=...)")
    modes = batch_modes(pc)
    out = {}
    for key, value in kwargs.items():
        if key in BATCH_DIMENSIONS_TP and torch.is_tensor(value) and key != "labels":
            for m in modes:
                value = comm.scatter(value, dim=BATCH_DIMENSIONS_TP[key], parallel_context=pc, parallel_mode=m)
        out[key] = value
    return (), out


class _Plan:
    """Per-mode split recipes."""

    def __init__(self, pc):
        self.pc = pc
        self.mode = pc.tensor_parallel_mode
        if self.mode == M.TENSOR_2D:
            self.row, self.col = M.TENSOR_2D_ROW, M.TENSOR_2D_COL
        elif self.mode == M.TENSOR_2P5D:
            self.row, self.col = M.TENSOR_2P5D_ROW, M.TENSOR_2P5D_COL

    # weight of a linear stored [out, in] (out_dim=0) or [in, out] (Conv1D)
    def linear_weight(self, out_dim, in_dim, parts):
        if self.mode in (M.TENSOR_2D, M.TENSOR_2P5D):
            return [Split(self.row, in_dim), Split(self.col, out_dim, parts)]
        return [Split(M.TENSOR_3D_OUTPUT, in_dim), Split(M.TENSOR_3D_INPUT, out_dim, parts), Split(M.TENSOR_3D_WEIGHT, out_dim)]

    def linear_bias(self, parts):
        if self.mode == M.TENSOR_2D:
            return [Split(self.row, 0, parts), Split(self.col, 0)]
        if self.mode == M.TENSOR_2P5D:
            return [Split(self.row, 0, parts)]
        return [Split(M.TENSOR_3D_INPUT, 0, parts)]

    def norm_param(self):
        if self.mode == M.TENSOR_2D:
            return [Split(self.row, 0), Split(self.col, 0)]
        if self.mode == M.TENSOR_2P5D:
            return [Split(self.row, 0)]
        return [Split(M.TENSOR_3D_OUTPUT, 0)]

    def vocab_embedding(self):
        if self.mode in (M.TENSOR_2D, M.TENSOR_2P5D):
            return [Split(self.col, 0), Split(self.row, 1)]
        return [Split(M.TENSOR_3D_INPUT, 0), Split(M.TENSOR_3D_WEIGHT, 0), Split(M.TENSOR_3D_OUTPUT, 1)]

    def other_embedding(self):
        if self.mode in (M.TENSOR_2D, M.TENSOR_2P5D):
            return [Split(self.row, 1), Split(self.col, 1)]
        return [Split(M.TENSOR_3D_OUTPUT, 1)]

    # which groups hold copies of a parameter whose gradient must therefore be summed
    def replicated_sync(self, kind):
        if self.mode == M.TENSOR_2D:
            return []
        if self.mode == M.TENSOR_2P5D:
            dep = [M.TENSOR_2P5D_DEP]
            return dep + ([M.TENSOR_2P5D_COL] if kind in ("bias", "norm") else [])
        if kind == "bias":
            return [M.TENSOR_3D_WEIGHT, M.TENSOR_3D_OUTPUT]
        if kind in ("norm", "other_embedding"):
            return [M.TENSOR_3D_WEIGHT, M.TENSOR_3D_INPUT]
        return []

    def linear_cls(self):
        return {M.TENSOR_2D: onn.Linear2D, M.TENSOR_2P5D: onn.Linear2p5D, M.TENSOR_3D: onn.Linear3D}[self.mode]

    def norm_cls(self):
        return {M.TENSOR_2D: onn.LayerNorm2D, M.TENSOR_2P5D: onn.LayerNorm2p5D, M.TENSOR_3D: onn.LayerNorm3D}[self.mode]

    def vocab_embedding_cls(self):
        return {M.TENSOR_2D: onn.VocabParallelEmbedding2D, M.TENSOR_2P5D: onn.VocabParallelEmbedding2p5D,
                M.TENSOR_3D: onn.VocabParallelEmbedding3D}[self.mode]

    def other_embedding_cls(self):
        return {M.TENSOR_2D: onn.Embedding2D, M.TENSOR_2P5D: onn.Embedding2p5D, M.TENSOR_3D: onn.Embedding3D}[self.mode]


def parallelize_nd(tp):
    """Shard ``tp.module`` for the context's N-D mode (called by ``TensorParallel.parallelize``)."""
    from .tensor_parallel import (_NORM_NAMES, _RMS_NAMES, _bare, _embedding_aliases, _is_conv1d, _is_linear_like,
                                  _keep_custom_embedding, _set_child, onn_marker)

    pc = tp.parallel_context
    module = tp.module
    mapping = tp._mapping()
    plan = _Plan(pc)
    mode = pc.tensor_parallel_mode
    is_oslo_model = isinstance(module, onn_marker())
    emb, head = tp._pad_vocab()
    tied = emb is not None and head is not None and head.weight is emb.weight
    new_tied = None
    dims = {}
    if mode in (M.TENSOR_2D, M.TENSOR_2P5D):
        dims["summa_dim" if mode == M.TENSOR_2D else "tesseract_dim"] = pc.summa_dim
        if mode == M.TENSOR_2P5D:
            dims["tesseract_dep"] = pc.tensor_parallel_depth
        feature_div = pc.summa_dim
    else:
        dims["cubic_dim"] = pc.cubic_dim
        feature_div = pc.cubic_dim

    cfg = getattr(module, "config", None)
    hidden_size = next((getattr(cfg, k) for k in ("hidden_size", "d_model", "n_embd", "dim") if isinstance(getattr(cfg, k, None), int)), None)
    feature_div_sq = feature_div * feature_div

    for attr in mapping.update_attrs(module):
        for m in module.modules():
            if hasattr(m, attr) and isinstance(getattr(m, attr), int) and m is not module:
                v = getattr(m, attr)
                if v % feature_div == 0:
                    tp._divided_attrs.append((m, attr, v))  # rolled back by deparallelize()
                    setattr(m, attr, v // feature_div)

    marked = set()

    def sync(p, kind):
        modes = plan.replicated_sync(kind)
        if modes and id(p) not in marked:
            marked.add(id(p))
            tp._mark_replicated(p, modes)

    def make_linear(child, name, w, b, gather_output):
        conv = _is_conv1d(child)
        out_dim, in_dim = (1, 0) if conv else (0, 1)
        new = _bare(plan.linear_cls(), in_features=w.shape[in_dim], out_features=w.shape[out_dim],
                    skip_bias_add=getattr(child, "skip_bias_add", False), gather_output=gather_output,
                    parallel_context=pc, reversed=conv, **dims)
        new.weight, new.bias = w, b
        if mode == M.TENSOR_2D:
            new.row_rank = pc.get_local_rank(M.TENSOR_2D_COL)
            new.col_rank = pc.get_local_rank(M.TENSOR_2D_ROW)
        return new

    from .tensor_parallel import _modules_inside_expert_blocks

    inside_experts = _modules_inside_expert_blocks(module)
    for name, child in list(module.named_modules()):
        if name == "" or (head is not None and child is head) or id(child) in inside_experts:
            continue
        if emb is not None and child is emb:
            full = child.weight.shape
            w = tp._shard_param(child.weight, ShardSpec(plan.vocab_embedding()), (module.orig_vocab_size, full[1]))
            new_tied = w if tied else None
            cls = plan.vocab_embedding_cls()
            new = _bare(cls, num_embeddings=w.shape[0], embedding_dim=w.shape[1], padding_idx=None, max_norm=None,
                        norm_type=2.0, scale_grad_by_freq=False, sparse=False, parallel_context=pc, **dims)
            if mode in (M.TENSOR_2D, M.TENSOR_2P5D):
                r = pc.get_local_rank(plan.col)
                per = full[0] // pc.summa_dim
                new.vocab_start_index, new.vocab_end_index = r * per, (r + 1) * per
            else:
                r = pc.get_local_rank(M.TENSOR_3D_INPUT)
                per = full[0] // pc.cubic_dim
                new.vocab_per_input = per
                new.vocab_start_index, new.vocab_end_index = r * per, (r + 1) * per
            new.weight = w
            new = _keep_custom_embedding(child, cls, new)
            aliases = _embedding_aliases(module, child)
            _set_child(module, name, new)
            for alias in aliases:
                _set_child(module, alias, new)  # encoder / decoder copies of the shared table
            continue
        if isinstance(child, nn.Embedding):
            if mapping.is_other(module, name):
                w = tp._shard_param(child.weight, ShardSpec(plan.other_embedding()))
                new = _bare(plan.other_embedding_cls(), num_embeddings=w.shape[0], embedding_dim=w.shape[1],
                            padding_idx=child.padding_idx, max_norm=None, norm_type=2.0, scale_grad_by_freq=False,
                            sparse=False, parallel_context=pc, **dims)
                new.weight = w
                sync(w, "other_embedding")
                _set_child(module, name, _keep_custom_embedding(child, plan.other_embedding_cls(), new))
            continue
        cname = child.__class__.__name__
        if cname in _NORM_NAMES + _RMS_NAMES:
            rms = cname in _RMS_NAMES
            full_dim = child.weight.shape[0]
            w = tp._shard_param(child.weight, ShardSpec(plan.norm_param()))
            b = None
            if getattr(child, "bias", None) is not None:
                b = tp._shard_param(child.bias, ShardSpec(plan.norm_param()))
            new = _bare(plan.norm_cls(), normalized_shape=full_dim, partitioned_dim=w.shape[0],
                        variance_epsilon=getattr(child, "eps", getattr(child, "variance_epsilon", 1e-5)), rms=rms,
                        parallel_context=pc, **dims)
            new.reduce_mode = {M.TENSOR_2D: M.TENSOR_2D_ROW, M.TENSOR_2P5D: M.TENSOR_2P5D_ROW,
                               M.TENSOR_3D: M.TENSOR_3D_OUTPUT}[mode]
            new.weight, new.bias = w, b
            sync(w, "norm")
            if b is not None:
                sync(b, "norm")
            _set_child(module, name, new)
            continue
        if not _is_linear_like(child):
            continue
        if not (mapping.is_column_parallel(module, name) or mapping.is_row_parallel(module, name)):
            # In the N-D layouts every activation between layers is sharded over features, so a linear the mapping does
            # not name (e.g. the transform in front of a masked-LM head) still has to take a feature shard.  It becomes an
            # N-D linear when it maps hidden -> hidden-like sizes that the grid divides; anything else is left alone.
            conv = _is_conv1d(child)
            o, i = (child.weight.shape[1], child.weight.shape[0]) if conv else child.weight.shape
            if hidden_size is None or i != hidden_size or o % feature_div_sq or i % feature_div_sq:
                continue
        conv = _is_conv1d(child)
        out_dim, in_dim = (1, 0) if conv else (0, 1)
        parts = mapping.get_combined_qkv_degree(child.weight) if mapping.is_combined_qkv_param(module, name) else 1
        w = tp._shard_param(child.weight, ShardSpec(plan.linear_weight(out_dim, in_dim, parts)))
        b = None
        if getattr(child, "bias", None) is not None:
            b = tp._shard_param(child.bias, ShardSpec(plan.linear_bias(parts)))
            sync(b, "bias")
        if mode == M.TENSOR_2P5D:
            sync(w, "weight")
        # between layers the N-D layouts keep activations sharded (the next norm / linear takes a shard), so the mapping's
        # gather_output, which in 1-D returns a column-parallel output to replicated form, only applies to heads
        _set_child(module, name, make_linear(child, name, w, b, False))

    if head is not None:
        name = next(n for n, m in module.named_modules() if m is head)
        conv = _is_conv1d(head)
        out_dim, in_dim = (1, 0) if conv else (0, 1)
        if tied:
            w = new_tied
        else:
            full = list(head.weight.shape)
            full[out_dim] = head.orig_num_classes
            w = tp._shard_param(head.weight, ShardSpec(plan.linear_weight(out_dim, in_dim, 1)), full)
        b = None
        if getattr(head, "bias", None) is not None:
            b = tp._shard_param(head.bias, ShardSpec(plan.linear_bias(1)), (head.orig_num_classes,))
            sync(b, "bias")
        if mode == M.TENSOR_2P5D:
            sync(w, "weight")
        # 3D has no vocab-parallel loss: logits are gathered and the plain loss runs on them
        gather = (mapping.is_gather_output(module, name) and not is_oslo_model) or mode == M.TENSOR_3D
        new = make_linear(head, name, w, b, gather)
        new.orig_num_classes = head.orig_num_classes
        _set_child(module, name, new)
    if emb is None:
        # No token table (vision models): the module that builds the first hidden state from pixels produces it whole, so
        # its output is cut to this rank's feature shard before the first sharded layer sees it.
        entry = next((m for n, m in module.named_modules() if n.split(".")[-1] == "embeddings"), None)
        if entry is not None:
            feature_mode = plan.row if mode in (M.TENSOR_2D, M.TENSOR_2P5D) else M.TENSOR_3D_OUTPUT

            def to_feature_shard(mod, inputs, output):
                if torch.is_tensor(output):
                    return comm.scatter(output, dim=-1, parallel_context=pc, parallel_mode=feature_mode)
                return output

            tp._entry_hooks = getattr(tp, "_entry_hooks", []) + [entry.register_forward_hook(to_feature_shard)]

    # task heads other than the vocabulary head (classifier, qa_outputs, seq_relationship, ...): they read the sharded hidden
    # state like any other linear; their few output classes are padded to what the grid divides, gathered, and cropped
    from ._sharding import pad_dim

    div = tp.get_divisible_by(pc)
    for name, child in list(module.named_modules()):
        if name == "" or child is head or not _is_linear_like(child) or not mapping.is_head(module, name):
            continue
        if isinstance(child, (onn.Linear2D, onn.Linear2p5D, onn.Linear3D)):
            continue
        conv = _is_conv1d(child)
        out_dim, in_dim = (1, 0) if conv else (0, 1)
        if child.weight.shape[in_dim] % feature_div_sq:
            continue
        classes = child.weight.shape[out_dim]
        full = list(child.weight.shape)
        child.weight.data = pad_dim(child.weight.data, out_dim, div)
        w = tp._shard_param(child.weight, ShardSpec(plan.linear_weight(out_dim, in_dim, 1)), full)
        b = None
        if getattr(child, "bias", None) is not None:
            child.bias.data = pad_dim(child.bias.data, 0, div)
            b = tp._shard_param(child.bias, ShardSpec(plan.linear_bias(1)), (classes,))
            sync(b, "bias")
        if mode == M.TENSOR_2P5D:
            sync(w, "weight")
        new = make_linear(child, name, w, b, True)
        new.orig_num_classes = classes
        _set_child(module, name, new)
    if mode == M.TENSOR_2P5D:
        # every parameter is replicated along the depth dimension
        for p in module.parameters():
            sync(p, "weight")
