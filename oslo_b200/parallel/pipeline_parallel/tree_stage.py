"""Pipeline stages for models that do not describe themselves with ``pipeline_units()``: the module tree is cut.

What the reference does for arbitrary models — walk the module tree, group it into segments of balanced cost and give
each segment to a pipeline rank (oslo/torch/nn/parallel/pipeline_parallel/_model_partitioner.py:79-284) — is done
here for the shape every transformer in Hugging Face has:

    [modules registered before the block list]  +  block_0 ... block_{L-1}  +  [modules registered after it]

The block list is the ``nn.ModuleList`` of same-class children that holds the most parameters.  The head part, the
blocks and the tail part are the units handed to :class:`ModelPartitioner`; a stage owns a contiguous range of them.

Execution keeps the model's OWN ``forward`` (mask construction, position ids, rotary tables and so on stay whatever
the model does) and makes the parts a stage does not own free of cost:

* a block of another stage returns its input;
* a parameterised leaf of another stage (embedding, head, final norm) returns zeros of the right shape without
  touching memory (an expanded scalar), or its input if it is a normalisation;
* the first block a stage owns gets the activation received from the previous stage in place of its input, and the
  output of the last block it owns is what goes to the next stage.

Stages other than the last are run without labels, so no loss is computed on placeholder logits.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from .partitioner import PipeUnit


def find_block_list(model: nn.Module) -> Tuple[str, nn.ModuleList]:
    lists = []
    for name, m in model.named_modules():
        if isinstance(m, nn.ModuleList) and len(m) >= 2 and len({type(c) for c in m}) == 1:
            lists.append((sum(p.numel() for p in m.parameters()), name, m))
    if not lists:
        raise TypeError(f"{type(model).__name__}: no list of repeated blocks found; define pipeline_units() instead")
    lists.sort(key=lambda t: -t[0])
    top = [(n, m) for _, n, m in lists if not any(n.startswith(o + ".") for _, o, _ in lists if o != n)]  # outermost lists only
    if len(top) >= 2 and {"encoder", "decoder"} <= {part for n, _ in top for part in n.split(".")}:
        raise TypeError(
            f"{type(model).__name__} has an encoder stack and a decoder stack ({', '.join(n for n, _ in top[:2])}); one "
            "activation crosses a stage boundary, which a model's own forward cannot express for two stacks.  The in-tree "
            "oslo_b200.models BART / mBART / T5 / mT5 classes load the same checkpoints and define pipeline_units().")
    return lists[0][1], lists[0][2]


def _leaf_modules_with_params(model: nn.Module, exclude: nn.Module) -> List[Tuple[str, nn.Module]]:
    inside = {id(m) for m in exclude.modules()}
    out = []
    for name, m in model.named_modules():
        if id(m) in inside:
            continue
        if any(True for _ in m.parameters(recurse=False)):
            out.append((name, m))
    return out


class TreeStage:
    """Built by ``PipelineParallel.parallelize`` for a model without ``pipeline_units()``."""

    def __init__(self, model: nn.Module):
        self.model = model
        self.block_name, self.blocks = find_block_list(model)
        names = [n for n, _ in model.named_modules()]
        pos = names.index(self.block_name)
        order = {n: i for i, n in enumerate(names)}
        leaves = _leaf_modules_with_params(model, self.blocks)
        # Registration order decides, with one correction: some models register the norm that runs AFTER the blocks before
        # the block list (OPT's ``final_layer_norm``).  A normalisation that is a sibling of the block list and is named as a
        # closing norm belongs to the tail; embedding norms (``layernorm_embedding``, ``embeddings.LayerNorm``) do not match.
        parent = self.block_name.rsplit(".", 1)[0] if "." in self.block_name else ""

        def closing_norm(name: str, mod: nn.Module) -> bool:
            leaf = name.rsplit(".", 1)[-1]
            sibling = (name.rsplit(".", 1)[0] if "." in name else "") == parent
            is_norm = "norm" in type(mod).__name__.lower()
            return sibling and is_norm and ("final" in leaf or leaf in ("ln_f", "norm", "layer_norm")) and "embed" not in leaf

        self.head = [(n, m) for n, m in leaves if order[n] < pos and not closing_norm(n, m)]
        self.tail = [(n, m) for n, m in leaves if order[n] > pos or (order[n] < pos and closing_norm(n, m))]
        self._inject: Optional[torch.Tensor] = None
        self._captured: Optional[torch.Tensor] = None
        self._orig_forward: Dict[int, object] = {}
        self.first_owned = self.last_owned = None
        self.is_first = self.is_last = True

    # ------------------------------------------------------------------ units
    def units(self) -> List[PipeUnit]:
        noop = lambda state: state
        u = [PipeUnit("head", [m for _, m in self.head], noop)]
        u += [PipeUnit(f"{self.block_name}.{i}", [b], noop) for i, b in enumerate(self.blocks)]
        u.append(PipeUnit("tail", [m for _, m in self.tail], noop))
        return u

    # ---------------------------------------------------------------- install
    def install(self, owned_units: range, num_units: int, stage: int, num_stages: int):
        """Stub what this stage does not own and hook the boundaries of what it does."""
        L = len(self.blocks)
        own_head, own_tail = 0 in owned_units, (num_units - 1) in owned_units
        owned_blocks = [i for i in range(L) if (i + 1) in owned_units]
        self.is_first, self.is_last = stage == 0, stage == num_stages - 1
        if not owned_blocks and not (own_head or own_tail):
            raise ValueError("a pipeline stage received no module")
        for i, b in enumerate(self.blocks):
            if i not in owned_blocks:
                self._stub(b, _identity_block)
        if not own_head:
            for _, m in self.head:
                self._stub(m, _placeholder_forward(m))
        if not own_tail:
            for _, m in self.tail:
                self._stub(m, _placeholder_forward(m))
        if owned_blocks:
            self.first_owned, self.last_owned = self.blocks[owned_blocks[0]], self.blocks[owned_blocks[-1]]
            if not self.is_first:
                self.first_owned.register_forward_pre_hook(self._pre_hook, with_kwargs=True)
            if not self.is_last:
                self.last_owned.register_forward_hook(self._post_hook)
        elif not self.is_first or not self.is_last:
            raise ValueError("every pipeline stage but a single one must own at least one block")

    def uninstall(self):
        """Give every stubbed module its own forward back and stop substituting activations (after deparallelize)."""
        for m in self.model.modules():
            if id(m) in self._orig_forward and "forward" in m.__dict__:
                del m.__dict__["forward"]
        self._orig_forward.clear()
        self.is_first = self.is_last = True
        self._handles_off = True

    def _stub(self, module: nn.Module, fn):
        self._orig_forward[id(module)] = module.forward
        module.forward = fn  # an instance attribute: called without ``self``

    def _pre_hook(self, module, args, kwargs):
        if self._inject is None or getattr(self, "_handles_off", False):
            return None
        h, self._inject = self._inject, None
        if args:
            return (h,) + tuple(args[1:]), kwargs
        kwargs = dict(kwargs)
        kwargs["hidden_states"] = h
        return args, kwargs

    def _post_hook(self, module, args, output):
        self._captured = output[0] if isinstance(output, (tuple, list)) else output
        return None

    # -------------------------------------------------------------------- run
    def run(self, state: dict) -> dict:
        kwargs = {k: v for k, v in state.items() if k not in ("hidden", "loss", "logits")}
        if not self.is_last:
            kwargs.pop("labels", None)
        self._inject = state.get("hidden") if not self.is_first else None
        self._captured = None
        out = self.model(**kwargs)
        if self.is_last:
            state["loss"] = getattr(out, "loss", None)
            state["logits"] = getattr(out, "logits", None)
        else:
            if self._captured is None:
                raise RuntimeError("the last block of this stage was not reached by the model's forward")
            state["hidden"] = self._captured
        return state


def _first_tensor(args, kwargs):
    for a in args:
        if torch.is_tensor(a):
            return a
    for k in ("hidden_states", "input", "inputs_embeds", "x"):
        if torch.is_tensor(kwargs.get(k)):
            return kwargs[k]
    for v in kwargs.values():
        if torch.is_tensor(v):
            return v
    raise TypeError("placeholder module called without a tensor argument")


def _identity_block(*args, **kwargs):
    """A block owned by another stage: hand the hidden states through untouched."""
    return _first_tensor(args, kwargs)


def _placeholder_forward(module: nn.Module):
    """Forward of a parameterised leaf that lives on another stage.  Its result is never used for anything that
    matters (the stage's real input arrives from its neighbour), so it only has to have the right shape and dtype."""
    dtype = next(module.parameters()).dtype
    if isinstance(module, nn.Embedding):
        dim = module.embedding_dim  # (the weight itself may already have been released on this stage)
        kind = type(module).__name__
        if "VocabParallel" not in kind:
            # the 2-D / 2.5-D position-style tables store h / q^2 columns and gather them to the h / q of the activations
            if "Embedding2D" in kind:
                dim *= module.summa_dim
            elif "Embedding2p5D" in kind:
                dim *= module.tesseract_dim

        def fwd(ids, *a, **k):
            if not torch.is_tensor(ids):  # position tables that take a shape (batch, seq) instead of ids
                shape, device = tuple(ids), module.weight.device
                return torch.zeros((), dtype=dtype, device=device).expand(*shape, dim)
            return torch.zeros((), dtype=dtype, device=ids.device).expand(*ids.shape, dim)

        return fwd
    out_features = getattr(module, "out_features", None) or getattr(module, "nf", None)
    if out_features is not None and not isinstance(module, (nn.LayerNorm,)):
        if hasattr(module, "orig_num_classes"):
            out_features = module.orig_num_classes

        def fwd(x, *a, **k):
            return torch.zeros((), dtype=x.dtype, device=x.device).expand(*x.shape[:-1], int(out_features))

        return fwd

    def fwd(*a, **k):  # normalisations and anything else: shape-preserving
        return _first_tensor(a, k)

    return fwd
