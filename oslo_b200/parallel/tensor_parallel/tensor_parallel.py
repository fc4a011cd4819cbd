"""``TensorParallel(module, parallel_context)``: shards a model for 1D / 2D / 2.5D / 3D tensor parallelism.

Usage (same as the reference)::

    model = TensorParallel(model, parallel_context)      # records the wrapper
    oslo_b200.ready(model, parallel_context)             # shards parameters, moves them to the device
    loss = model(input_ids=..., labels=...).loss

Mechanism: parameters are sliced according to a per-parameter :class:`ShardSpec` computed from the name mapping,
and each affected sub-module is REPLACED by its parallel counterpart (``ColLinear1D``, ``Linear2D`` ...) holding
the slice — attribute names, hence state-dict keys, are unchanged.  ``deparallelize()`` merges every shard
back (all-gathers driven by the spec), restores plain layers and crops the vocabulary padding.

``sequence_parallel=True`` (1D only, not in the reference) keeps activations token-sharded between the
linears: column linears all-gather -> GEMM, row linears GEMM -> reduce-scatter, fused on CUDA.

Parity: oslo/torch/nn/parallel/tensor_parallel/tensor_parallel.py:33-236 and _1d/_wrapper.py:55-567.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

import oslo_b200.nn as onn
from oslo_b200.distributed import ParallelMode, comm
from oslo_b200.parallel.utils import ParallelWrapper, add_wrapper, get_parallel_context, unwrap_parallel

from ._sharding import ShardSpec, Split, merge, pad_dim, shard
from .mapping import TensorParallelMapping

_NORM_NAMES = ("LayerNorm", "FusedLayerNorm", "MixedFusedLayerNorm", "LayerNorm1D")
_RMS_NAMES = ("FusedRMSNorm", "MixedFusedRMSNorm", "RMSNorm1D", "LlamaRMSNorm", "T5LayerNorm")


def _is_linear_like(m) -> bool:
    return isinstance(m, nn.Linear) or m.__class__.__name__ == "Conv1D"


def _is_conv1d(m) -> bool:
    return m.__class__.__name__ == "Conv1D"


def _set_child(root: nn.Module, dotted: str, new: nn.Module):
    """Put ``new`` where ``dotted`` is, and everywhere else the same module object is registered (a table shared by an
    encoder and a decoder is one object under several names; ``named_modules`` reports only the first)."""
    parent = root
    parts = dotted.split(".")
    for p in parts[:-1]:
        parent = getattr(parent, p)
    old = getattr(parent, parts[-1], None)
    setattr(parent, parts[-1], new)
    if isinstance(old, nn.Module):
        for m in root.modules():
            for key, sub in m._modules.items():
                if sub is old:
                    m._modules[key] = new


def _modules_inside_expert_blocks(root: nn.Module) -> set:
    """Routers and experts of a mixture-of-experts layer are placed by the expert-parallel wrapper; the tensor-parallel
    wrapper leaves everything inside such a block alone (a router called ``...c_fc.gate.wg`` is not the ``c_fc`` linear the
    mapping names)."""
    try:
        from oslo_b200.parallel.expert_parallel.layers import ExpertParallelBehindBlock, ExpertParallelFrontBlock
    except ImportError:
        return set()
    out = set()
    for m in root.modules():
        if isinstance(m, (ExpertParallelFrontBlock, ExpertParallelBehindBlock)):
            out.update(id(d) for d in m.modules())
    return out


def _embedding_aliases(root: nn.Module, emb: nn.Module):
    """Names of the OTHER embedding modules that hold ``emb``'s weight parameter (libraries that give an encoder and a
    decoder their own ``nn.Embedding`` tied to the shared table): they must become the same sharded module."""
    w = getattr(emb, "weight", None)
    return [n for n, m in root.named_modules() if m is not emb and isinstance(m, nn.Embedding) and getattr(m, "weight", None) is w]


def _keep_custom_embedding(child: nn.Module, parallel_cls, new: nn.Module) -> nn.Module:
    """Libraries subclass ``nn.Embedding`` to do something around the lookup (scale the result, turn a shape or a mask into
    position ids, add an offset) and then call ``super().forward(ids)``.  Swapping such a module for a plain parallel
    embedding would drop that behaviour, so the replacement's class becomes ``(original subclass, parallel class)``: the
    original ``forward`` still runs and its ``super().forward`` now reaches the parallel lookup.  Plain attributes of the
    original (scale factors, offsets) are carried over."""
    cls = type(child)
    if cls is nn.Embedding or not isinstance(child, nn.Embedding) or cls.forward is nn.Embedding.forward:
        return new
    new.__class__ = type(f"{parallel_cls.__name__}For{cls.__name__}", (cls, parallel_cls), {})
    for key, value in child.__dict__.items():
        if key not in new.__dict__ and not key.startswith("_"):
            new.__dict__[key] = value
    return new


def _bare(cls, **attrs):
    """Instantiate ``cls`` without running its constructor (no throw-away parameter allocation)."""
    obj = cls.__new__(cls)
    nn.Module.__init__(obj)
    for k, v in attrs.items():
        setattr(obj, k, v)
    return obj


class SequenceParallelState:
    """Which dim of ``[batch, seq, hidden]`` activations is sharded between the linears (set per forward)."""

    def __init__(self, pc):
        self.pc = pc
        self.dim = 0

    def configure(self, batch: int, seq: int):
        tp = self.pc.get_world_size(ParallelMode.TENSOR_1D)
        self.full = (batch, seq)
        if batch % tp == 0:
            self.dim = 0
        elif batch == 1 and seq % tp == 0:
            self.dim = 1
        else:
            raise ValueError(
                f"sequence parallelism needs batch ({batch}) divisible by the tensor-parallel size ({tp}), "
                f"or batch 1 with seq ({seq}) divisible by it")

    def shard(self, t):
        return comm.scatter(t, dim=self.dim, parallel_context=self.pc, parallel_mode=ParallelMode.TENSOR_1D)

    def shard_if_full(self, t):
        """Cut ``t`` to this rank's share when it still spans the whole batch / sequence along the sharded dimension (a
        size-1 dimension that broadcasts against the shard is left alone)."""
        full = getattr(self, "full", None)
        if full is None or not torch.is_tensor(t) or t.dim() <= self.dim:
            return t
        size = t.shape[self.dim]
        if size != full[self.dim] and not (self.dim == 1 and size in getattr(self, "other_lengths", ())):
            return t
        if self.pc.get_world_size(ParallelMode.TENSOR_1D) == 1:
            return t
        return self.shard(t)


class TensorParallel(ParallelWrapper):
    parallelism_priority = 0

    def __init__(self, module: nn.Module, parallel_context=None, mapping: Optional[dict] = None,
                 module_args: Optional[dict] = None, sequence_parallel: bool = False, vocab_parallel_loss: bool = False):
        super().__init__()
        self.module = module
        self.parallel_context = get_parallel_context(module, parallel_context)
        self.sequence_parallel = sequence_parallel
        #: stock Hugging Face language models (1-D mode): keep the head's logits sharded over the vocabulary and compute
        #: the loss with the vocab-parallel cross-entropy instead of gathering [tokens, vocab] logits on every rank (what
        #: the reference's model forks do, oslo/transformers/models/gpt2/modeling_gpt2.py:845-875).  ``output.logits``
        #: then holds this rank's vocabulary slice.
        self.vocab_parallel_loss = vocab_parallel_loss
        self._mapping_arg = mapping
        self.module_args = module_args
        mode = self.parallel_context.tensor_parallel_mode
        if sequence_parallel and mode != ParallelMode.TENSOR_1D:
            raise ValueError("sequence_parallel=True is only defined for 1D tensor parallelism")
        if sequence_parallel and type(module).__module__.startswith("transformers.") \
                and not type(module).__name__.startswith(("GPT2", "GPTJ")):
            # Between blocks the activations are token shards and the column-parallel projections return the gathered
            # sequence.  Most Hugging Face attention modules take (batch, seq) from their INPUT and reshape the projections
            # with it, which silently folds tokens into heads; GPT-2 and GPT-J take the shape from the projections.
            raise NotImplementedError(
                f"sequence_parallel=True is not supported for transformers' {type(module).__name__}: its attention reshapes "
                "the projections with the input's sequence length.  Use the in-tree model of the same family "
                "(oslo_b200.models; it loads the same checkpoint) or sequence_parallel=False.")
        self.sp_state = SequenceParallelState(self.parallel_context) if sequence_parallel else None
        self._sp_params = []
        self._sp_callback_queued = False
        self._divided_attrs = []  # (module, attribute, value before the division by the tensor-parallel size)
        add_wrapper(module, ParallelMode.TENSOR, self)

    # ------------------------------------------------------------------ forward
    def forward(self, *args, **kwargs):
        pc = self.parallel_context
        mode = pc.tensor_parallel_mode
        if self.sp_state is not None:
            ids = kwargs.get("input_ids", args[0] if args else None)
            if ids is not None and ids.dim() >= 2:
                self.sp_state.configure(ids.shape[0], ids.shape[1])
                # a decoder runs on its own sequence length: position tables looked up for it are cut the same way
                other = kwargs.get("decoder_input_ids", kwargs.get("labels"))
                self.sp_state.other_lengths = {other.shape[1]} if other is not None and other.dim() >= 2 else set()
        elif getattr(self, "_parallelized", False) and mode != ParallelMode.TENSOR_1D and pc.tensor_parallel_size > 1:
            from ._wrapper_nd import scatter_batch_inputs

            args, kwargs = scatter_batch_inputs(self.module, args, kwargs, pc)
        if self._vp_loss_active and kwargs.get("labels") is not None:
            return self._forward_vocab_parallel_loss(args, kwargs)
        return self.module(*args, **kwargs)

    @property
    def _vp_loss_active(self) -> bool:
        pc = self.parallel_context
        return (self.vocab_parallel_loss and getattr(self, "_parallelized", False) and pc.tensor_parallel_size > 1
                and pc.tensor_parallel_mode == ParallelMode.TENSOR_1D and not isinstance(self.module, onn_marker()))

    def _forward_vocab_parallel_loss(self, args, kwargs):
        """Run the model without labels (its head leaves the logits sharded), then the vocab-parallel cross-entropy:
        next-token targets for causal language models, the labels as they are for masked ones."""
        from oslo_b200.models.losses import shift_labels

        kwargs = dict(kwargs)
        labels = kwargs.pop("labels")
        if getattr(getattr(self.module, "config", None), "is_encoder_decoder", False) and kwargs.get("decoder_input_ids") is None \
                and kwargs.get("decoder_inputs_embeds") is None:
            # the model would have derived the decoder inputs from the labels it no longer receives
            make = getattr(self.module, "prepare_decoder_input_ids_from_labels", None) or getattr(self.module, "_shift_right", None) \
                or getattr(self.module, "_shift", None)
            if make is None:
                raise ValueError("give decoder_input_ids: this model cannot derive them from labels")
            kwargs["decoder_input_ids"] = make(labels)
        out = self.module(*args, **kwargs)
        logits = out.logits if hasattr(out, "logits") else out[0]
        name = type(self.module).__name__
        causal = name.endswith(("ForCausalLM", "LMHeadModel")) or "CausalLM" in name
        targets = shift_labels(labels) if causal else labels
        fn = onn.VocabParallelCrossEntropyLoss1D(parallel_context=self.parallel_context, ignore_index=-100)
        fn.orig_vocab_size = getattr(self.module, "orig_vocab_size", self.module.config.vocab_size)
        loss = fn(logits, targets.to(logits.device))
        if hasattr(out, "loss"):
            out.loss = loss
            return out
        return (loss,) + tuple(out)

    # ------------------------------------------------------------ parallelize
    def _mapping(self):
        from oslo_b200.transformers.mapping_utils import _TensorParallelMapping

        return _TensorParallelMapping(self._mapping_arg)

    @torch.no_grad()
    def parallelize(self):
        pc = self.parallel_context
        module = self.module
        module.parallel_context = pc
        for m in module.modules():
            if hasattr(m, "config") and not hasattr(m, "parallel_context"):
                m.parallel_context = pc
        if pc.tensor_parallel_size == 1:
            return
        mode = pc.tensor_parallel_mode
        if mode == ParallelMode.TENSOR_1D:
            self._parallelize_1d()
        else:
            from ._wrapper_nd import parallelize_nd

            parallelize_nd(self)

    @staticmethod
    def get_divisible_by(pc) -> int:
        mode = pc.tensor_parallel_mode
        if mode == ParallelMode.TENSOR_1D:
            return pc.tensor_parallel_size
        if mode == ParallelMode.TENSOR_2D:
            return pc.summa_dim ** 2
        if mode == ParallelMode.TENSOR_2P5D:
            return pc.summa_dim
        if mode == ParallelMode.TENSOR_3D:
            return pc.cubic_dim ** 2
        return 1

    def _pad_vocab(self):
        """Pad the input embedding (and an untied head) to a multiple of the mode's divisor; remember the true size."""
        module = self.module
        div = self.get_divisible_by(self.parallel_context)
        emb = module.get_input_embeddings() if hasattr(module, "get_input_embeddings") else None
        if emb is None or not isinstance(getattr(emb, "weight", None), torch.Tensor) or emb.weight.dim() != 2:
            return None, None  # no token table (e.g. a vision model's patch projection): nothing to pad
        head = module.get_output_embeddings() if hasattr(module, "get_output_embeddings") else None
        tied = head is not None and head.weight is emb.weight
        orig = emb.weight.shape[0]
        module.orig_vocab_size = orig
        if orig % div:
            emb.weight.data = pad_dim(emb.weight.data, 0, div)
            emb.num_embeddings = emb.weight.shape[0]
        module.padded_vocab_size = emb.weight.shape[0]
        if head is not None and not tied:
            w = head.weight
            out_dim = 1 if _is_conv1d(head) else 0
            head.orig_num_classes = w.shape[out_dim]
            if w.shape[out_dim] % div:
                head.weight.data = pad_dim(w.data, out_dim, div)
                if getattr(head, "bias", None) is not None:
                    head.bias.data = pad_dim(head.bias.data, 0, div)
                if hasattr(head, "out_features"):
                    head.out_features = head.weight.shape[out_dim]
        elif head is not None:
            head.orig_num_classes = orig
        return emb, head

    def _stamp(self, p: nn.Parameter, spec: ShardSpec):
        pc = self.parallel_context
        p.oslo_shard = spec
        p.oslo_parallel = {s.mode: pc.get_local_rank(s.mode) for s in spec.splits}

    def _shard_param(self, p: nn.Parameter, spec: ShardSpec, full_shape=None) -> nn.Parameter:
        spec.full_shape = tuple(full_shape if full_shape is not None else p.shape)
        new = nn.Parameter(shard(p.data, spec, self.parallel_context), requires_grad=p.requires_grad)
        self._stamp(new, spec)
        return new

    def _parallelize_1d(self):
        pc = self.parallel_context
        module = self.module
        mapping = self._mapping()
        tp = pc.tensor_parallel_size
        M1 = ParallelMode.TENSOR_1D
        sp = self.sequence_parallel
        is_oslo_model = isinstance(module, onn_marker())
        emb, head = self._pad_vocab()
        tied_weight = emb.weight if (emb is not None and head is not None and head.weight is emb.weight) else None
        new_tied = None

        # HF-style models divide per-rank head counts etc.
        for attr in mapping.update_attrs(module):
            for m in module.modules():
                if hasattr(m, attr) and isinstance(getattr(m, attr), int) and not isinstance(m, type(module)):
                    v = getattr(m, attr)
                    if v % tp == 0:
                        self._divided_attrs.append((m, attr, v))  # rolled back by deparallelize()
                        setattr(m, attr, v // tp)

        inside_experts = _modules_inside_expert_blocks(module)
        for name, child in list(module.named_modules()):
            if name == "" or id(child) in inside_experts:
                continue
            if emb is not None and child is emb:
                full = child.weight.shape
                w = self._shard_param(child.weight, ShardSpec([Split(M1, 0)]), (module.orig_vocab_size, full[1]))
                if tied_weight is not None:
                    new_tied = w
                rank = pc.get_local_rank(M1)
                new = _bare(onn.VocabParallelEmbedding1D, num_embeddings=full[0] // tp, embedding_dim=full[1],
                            padding_idx=None, max_norm=None, norm_type=2.0, scale_grad_by_freq=False, sparse=False,
                            parallel_context=pc, sequence_parallel=sp, world_size=tp,
                            vocab_start_index=rank * (full[0] // tp), vocab_end_index=(rank + 1) * (full[0] // tp),
                            sequence_parallel_state=self.sp_state)
                new.weight = w
                new = _keep_custom_embedding(child, onn.VocabParallelEmbedding1D, new)
                for alias in _embedding_aliases(module, child):
                    _set_child(module, alias, new)  # other modules built around the same table (encoder / decoder copies)
                _set_child(module, name, new)
                continue
            if head is not None and child is head:
                continue  # after the loop (needs the tied weight)
            if not _is_linear_like(child):
                if isinstance(child, nn.Embedding) and mapping.is_other(module, name) and tp > 1 \
                        and not mapping.is_gather_output(module, name) and child.embedding_dim % tp == 0:
                    # a table with one column per head (T5's relative attention bias): every rank keeps its heads' columns
                    w = self._shard_param(child.weight, ShardSpec([Split(M1, 1)]))
                    new = _bare(onn.Embedding1D, num_embeddings=w.shape[0], embedding_dim=w.shape[1], padding_idx=None,
                                max_norm=None, norm_type=2.0, scale_grad_by_freq=False, sparse=False, parallel_context=pc,
                                world_size=tp, gather_output=False)
                    new.weight = w
                    _set_child(module, name, new)
                elif isinstance(child, nn.Embedding) and mapping.is_other(module, name) and sp:
                    self._mark_sp(child)
                    if not isinstance(module, onn_marker()) or getattr(module, "sequence_parallel_shards_other_embeddings", True):
                        # position / token-type tables are looked up for the whole batch; what is added to the token-sharded
                        # word embeddings must be this rank's share
                        state = self.sp_state
                        handle = child.register_forward_hook(lambda mod, inputs, out, state=state: state.shard_if_full(out))
                        self._entry_hooks = getattr(self, "_entry_hooks", []) + [handle]  # removed by deparallelize()
                elif child.__class__.__name__ in _NORM_NAMES + _RMS_NAMES:
                    if sp:
                        self._mark_sp(child)
                continue
            conv = _is_conv1d(child)
            out_dim, in_dim = (1, 0) if conv else (0, 1)
            has_bias = getattr(child, "bias", None) is not None
            skip = getattr(child, "skip_bias_add", False)
            if sp and mapping.is_column_parallel(module, name) and mapping.is_gather_output(module, name):
                # A column-parallel linear whose output is gathered again computes, in the end, the whole product on every
                # rank.  Under sequence parallelism its input is a token shard, so the same result per token comes from
                # simply keeping the layer whole and applying it to the shard: the activation stays token-sharded for
                # whatever follows (norm, head), and nothing is gathered twice.  Its gradients are partial sums over tokens.
                self._mark_sp(child)
                continue
            if mapping.is_column_parallel(module, name):
                parts = mapping.get_combined_qkv_degree(child.weight) if mapping.is_combined_qkv_param(module, name) else 1
                w = self._shard_param(child.weight, ShardSpec([Split(M1, out_dim, parts)]))
                b = self._shard_param(child.bias, ShardSpec([Split(M1, 0, parts)])) if has_bias else None
                new = _bare(onn.ColLinear1D, in_features=w.shape[in_dim], out_features=w.shape[out_dim],
                            skip_bias_add=skip, gather_output=mapping.is_gather_output(module, name),
                            parallel_context=pc, sequence_parallel=sp, world_size=tp, reversed=conv,
                            sequence_parallel_state=self.sp_state)
                new.weight, new.bias = w, b
                _set_child(module, name, new)
            elif mapping.is_row_parallel(module, name):
                w = self._shard_param(child.weight, ShardSpec([Split(M1, in_dim)]))
                new = _bare(onn.RowLinear1D, in_features=w.shape[in_dim], out_features=w.shape[out_dim],
                            skip_bias_add=skip, parallel_input=True, parallel_context=pc, sequence_parallel=sp,
                            world_size=tp, reversed=conv, sequence_parallel_state=self.sp_state)
                new.weight = w
                new.bias = child.bias if has_bias else None
                if has_bias and sp:
                    self._mark_sp_param(new.bias)
                _set_child(module, name, new)

        if head is not None:
            name = next(n for n, m in module.named_modules() if m is head)
            conv = _is_conv1d(head)
            out_dim, in_dim = (1, 0) if conv else (0, 1)
            if tied_weight is not None:
                w = new_tied
            else:
                full = list(head.weight.shape)
                full[out_dim] = head.orig_num_classes
                w = self._shard_param(head.weight, ShardSpec([Split(M1, out_dim)]), full)
            has_bias = getattr(head, "bias", None) is not None
            b = None
            if has_bias:
                b = self._shard_param(head.bias, ShardSpec([Split(M1, 0)]), (head.orig_num_classes,))
            gather = mapping.is_gather_output(module, name) and not is_oslo_model
            if self.vocab_parallel_loss and head is getattr(module, "get_output_embeddings", lambda: None)():
                gather = False  # the loss consumes the vocabulary shards directly
                flb = getattr(module, "final_logits_bias", None)
                if torch.is_tensor(flb) and flb.shape[-1] == head.orig_num_classes:
                    # a per-token bias added to the logits (BART): this rank adds its slice to its slice of the logits
                    self._saved_buffers = getattr(self, "_saved_buffers", []) + [(module, "final_logits_bias", flb)]
                    per = w.shape[out_dim]
                    padded = torch.zeros(*flb.shape[:-1], per * tp, dtype=flb.dtype, device=flb.device)
                    padded[..., : flb.shape[-1]] = flb
                    rank_ = pc.get_local_rank(M1)
                    module.final_logits_bias = padded[..., rank_ * per : (rank_ + 1) * per].clone()
            new = _bare(onn.ColLinear1D, in_features=w.shape[in_dim], out_features=w.shape[out_dim],
                        skip_bias_add=False, gather_output=gather, parallel_context=pc, sequence_parallel=sp,
                        world_size=tp, reversed=conv, sequence_parallel_state=self.sp_state)
            new.weight, new.bias = w, b
            new.orig_num_classes = head.orig_num_classes
            _set_child(module, name, new)
        for m in module.modules():
            if self.sp_state is not None and hasattr(m, "config"):
                m.sequence_parallel_state = self.sp_state
        if self.sp_state is not None:
            for m in module.modules():
                if m.__class__.__name__.endswith(("Attention", "MLP", "Layer", "Block", "Model")):
                    m.sequence_parallel_state = self.sp_state

    # ------------------------------------------ replicated-parameter gradient sync
    def _mark_replicated(self, p: nn.Parameter, modes):
        """``p`` is held identically by every rank of ``modes`` but sees rank-specific data: sum its gradient over
        those groups at the end of backward (one flattened all-reduce per distinct group list)."""
        modes = tuple(modes)
        if not hasattr(self, "_replicated"):
            self._replicated = {}
            self._rep_callback_queued = False
        if any(p is q for q in self._replicated.get(modes, [])):
            return
        self._replicated.setdefault(modes, []).append(p)
        p.register_post_accumulate_grad_hook(self._rep_hook)

    def _rep_hook(self, p):
        if not self._rep_callback_queued:
            self._rep_callback_queued = True
            torch.autograd.Variable._execution_engine.queue_callback(self._reduce_replicated_grads)

    def _reduce_replicated_grads(self):
        self._rep_callback_queued = False
        pc = self.parallel_context
        for modes, params in self._replicated.items():
            grads = [p.grad for p in params if p.grad is not None]
            by_dtype = {}
            for g in grads:
                by_dtype.setdefault(g.dtype, []).append(g)
            for gs in by_dtype.values():
                flat = torch.cat([g.reshape(-1) for g in gs])
                for m in modes:
                    comm.all_reduce(flat, parallel_context=pc, parallel_mode=m)
                off = 0
                for g in gs:
                    n = g.numel()
                    g.copy_(flat[off : off + n].view_as(g))
                    off += n

    # ---------------------------------------- sequence-parallel gradient sync
    def _mark_sp(self, m: nn.Module):
        for p in m.parameters(recurse=False):
            self._mark_sp_param(p)

    def _mark_sp_param(self, p: nn.Parameter):
        """Gradients of parameters applied to token-sharded activations are partial sums: all-reduce them once,
        flattened, at the end of backward."""
        if getattr(p, "sequence_parallel_grad", False):
            return
        p.sequence_parallel_grad = True
        self._sp_params.append(p)
        p.register_post_accumulate_grad_hook(self._sp_hook)

    def _sp_hook(self, p):
        if not self._sp_callback_queued:
            self._sp_callback_queued = True
            torch.autograd.Variable._execution_engine.queue_callback(self._reduce_sp_grads)

    def _reduce_sp_grads(self):
        self._sp_callback_queued = False
        grads = [p.grad for p in self._sp_params if p.grad is not None]
        if not grads:
            return
        pc = self.parallel_context
        by_dtype = {}
        for g in grads:
            by_dtype.setdefault(g.dtype, []).append(g)
        for gs in by_dtype.values():
            flat = torch.cat([g.reshape(-1) for g in gs])
            comm.all_reduce(flat, parallel_context=pc, parallel_mode=ParallelMode.TENSOR_1D)
            off = 0
            for g in gs:
                n = g.numel()
                g.copy_(flat[off : off + n].view_as(g))
                off += n

    # ---------------------------------------------------------- deparallelize
    @torch.no_grad()
    def deparallelize(self):
        """Merge every shard back into full tensors and restore plain layers (collective over the TP group)."""
        pc = self.parallel_context
        module = self.module
        if pc.tensor_parallel_size == 1:
            return
        for handle in getattr(self, "_entry_hooks", []):
            handle.remove()
        self._entry_hooks = []
        for owner, name, value in getattr(self, "_saved_buffers", []):
            setattr(owner, name, value)
        self._saved_buffers = []
        merged = {}
        for name, child in list(module.named_modules()):
            if name == "":
                continue
            params = dict(child.named_parameters(recurse=False))
            if not any(hasattr(p, "oslo_shard") for p in params.values()):
                continue
            full = {}
            for pname, p in params.items():
                if hasattr(p, "oslo_shard"):
                    if id(p) not in merged:
                        merged[id(p)] = nn.Parameter(merge(p.data, p.oslo_shard, pc), requires_grad=p.requires_grad)
                    full[pname] = merged[id(p)]
                else:
                    full[pname] = p
            _set_child(module, name, _restore_plain(child, full))
        if hasattr(module, "orig_vocab_size"):
            module.padded_vocab_size = module.orig_vocab_size
        # per-module arguments that were divided by the tensor-parallel size (head counts, split sizes, ...) get their
        # original values back (the reference's _rollback_mp_arguments, .../_1d/_wrapper.py)
        for m, attr, value in reversed(self._divided_attrs):
            setattr(m, attr, value)
        self._divided_attrs = []
        # gradient-sync bookkeeping refers to parameters that no longer exist
        self._sp_params = []
        self._sp_callback_queued = False
        if hasattr(self, "_replicated"):
            self._replicated = {}
            self._rep_callback_queued = False
        for m in module.modules():
            if getattr(m, "sequence_parallel_state", None) is not None:
                m.sequence_parallel_state = None
        self.sp_state = None
        self.sequence_parallel = False
        self._parallelized = False


def onn_marker():
    from oslo_b200.models.modeling_utils import OsloModel

    return OsloModel


def _restore_plain(child: nn.Module, params: dict) -> nn.Module:
    """Plain (unsharded) equivalent of a parallel layer, adopting the merged parameters."""
    w = params.get("weight")
    b = params.get("bias")
    if isinstance(child, nn.Embedding):
        # an embedding subclass with its own forward (see _keep_custom_embedding) gets that class back
        custom = next((c for c in type(child).__mro__[1:] if issubclass(c, nn.Embedding) and c is not nn.Embedding
                       and not c.__module__.startswith("oslo_b200.nn")), nn.Embedding)
        new = _bare(custom, num_embeddings=w.shape[0], embedding_dim=w.shape[1], padding_idx=getattr(child, "padding_idx", None),
                    max_norm=None, norm_type=2.0, scale_grad_by_freq=False, sparse=False)
        if custom is not nn.Embedding:
            for key, value in child.__dict__.items():
                if key not in new.__dict__ and not key.startswith("_") and key not in (
                        "parallel_context", "vocab_start_index", "vocab_end_index", "world_size", "sequence_parallel",
                        "sequence_parallel_state", "summa_dim", "tesseract_dim", "tesseract_dep", "cubic_dim", "vocab_per_input"):
                    new.__dict__[key] = value
        new.weight = w
        return new
    if isinstance(child, nn.Linear):
        if getattr(child, "reversed", False):
            new = _bare(onn.Conv1D, nf=w.shape[1], skip_bias_add=getattr(child, "skip_bias_add", False))
        else:
            new = _bare(onn.Linear, in_features=w.shape[1], out_features=w.shape[0],
                        skip_bias_add=getattr(child, "skip_bias_add", False))
        new.weight, new.bias = w, b
        return new
    if child.__class__.__name__.startswith("LayerNorm") and getattr(child, "rms", False):
        new = _bare(onn.FusedRMSNorm, normalized_shape=(w.shape[0],), eps=getattr(child, "variance_epsilon", 1e-6),
                    elementwise_affine=True)
        new.weight = w
        return new
    if child.__class__.__name__.startswith("LayerNorm"):
        new = _bare(onn.FusedLayerNorm, normalized_shape=(w.shape[0],), eps=getattr(child, "variance_epsilon", 1e-5),
                    elementwise_affine=True)
        new.weight, new.bias = w, b
        return new
    for k, v in params.items():
        setattr(child, k, v)
    return child
