"""A small static-graph runtime: declare the operators of a model once against maximum shapes, plan ONE arena for all
intermediate tensors from their lifetimes, then run any batch that fits without allocating.

Counterpart of the ``lsflow`` executor of the reference's LightSeq subset (oslo/lightseq2/csrc/lsflow/{context,node,
variable,layer,manager}.cpp: ``Context`` with a layer / node registry, ``Variable`` with maximum size, ``Operator`` nodes,
a dry run that records lifetimes and a ``MemoryManager`` that packs them into one buffer).  Here:

* :class:`Context` owns the node list, the plan (``csrc/cpu/memory_planner.cpp`` through
  :func:`oslo_b200.lightseq.memory_planner.plan`) and the arena tensor;
* :class:`Variable` is a symbolic tensor with a maximum shape; at run time its ``value`` is a view into the arena with the
  current leading dimension (graph inputs and parameters are bound tensors, outside the arena);
* :class:`Operator` subclasses declare their outputs when applied (graph construction) and compute into the output views
  when the context runs.  Since shapes and addresses are fixed after ``build()``, a run is a fixed sequence of kernel
  launches on fixed buffers (it can be captured in a CUDA graph by the caller).

Only inference (forward) graphs are built here; training goes through autograd modules.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .memory_planner import check, plan

_ALIGN = 256


class Variable:
    """Symbolic tensor.  ``max_shape[0]`` is the dimension that may shrink at run time (tokens); the others are fixed."""

    def __init__(self, ctx: "Context", name: str, max_shape: Sequence[int], dtype: torch.dtype, external: bool = False):
        self.ctx, self.name, self.max_shape, self.dtype, self.external = ctx, name, tuple(int(s) for s in max_shape), dtype, external
        self.producer: Optional["Operator"] = None
        self.first_use = self.last_use = -1
        self.offset = -1
        self.value: Optional[torch.Tensor] = None
        ctx._variables.append(self)

    @property
    def max_bytes(self) -> int:
        return math.prod(self.max_shape) * torch.empty((), dtype=self.dtype).element_size()

    def view(self, lead: int) -> torch.Tensor:
        shape = (lead,) + self.max_shape[1:]
        n = math.prod(shape)
        esz = torch.empty((), dtype=self.dtype).element_size()
        return self.ctx.arena[self.offset : self.offset + n * esz].view(self.dtype).view(shape)


class Operator:
    """One node.  ``__call__`` (graph construction) registers inputs and returns the output variable(s); ``run`` computes
    into ``out.value`` from ``inp.value``."""

    def __init__(self, ctx: "Context", name: str):
        self.ctx, self.name = ctx, name
        self.inputs: List[Variable] = []
        self.outputs: List[Variable] = []

    def _register(self, inputs: Sequence[Variable], outputs: Sequence[Variable]):
        if self.ctx.built:
            raise RuntimeError("the graph is frozen after build()")
        self.inputs, self.outputs = list(inputs), list(outputs)
        step = len(self.ctx._nodes)
        for v in inputs:
            if not v.external:
                v.last_use = max(v.last_use, step)
        for v in outputs:
            v.producer, v.first_use, v.last_use = self, step, step
        self.ctx._nodes.append(self)

    def run(self, lead: int):
        raise NotImplementedError


class LinearOp(Operator):
    """``out = act(x @ W^T + b)``; ``act`` in {None, "gelu", "relu"} (GELU rides in the GEMM epilogue on CUDA)."""

    def __init__(self, ctx, name, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, act: Optional[str] = None):
        super().__init__(ctx, name)
        self.weight, self.bias, self.act = weight, bias, act

    def __call__(self, x: Variable) -> Variable:
        out = Variable(self.ctx, self.name + ".out", (x.max_shape[0], self.weight.shape[0]), x.dtype)
        self._register([x], [out])
        return out

    def run(self, lead):
        from oslo_b200.ops.gemm import gemm, supported

        x, out = self.inputs[0].value, self.outputs[0].value
        if supported(x, self.weight) and x.shape[-1] % 8 == 0 and self.weight.shape[0] % 8 == 0:
            gemm(x, self.weight, bias=self.bias, epilogue="gelu" if self.act == "gelu" else ("bias" if self.bias is not None else None),
                 out=out)
            if self.act == "relu":
                out.relu_()
            return
        torch.matmul(x, self.weight.t(), out=out)
        if self.bias is not None:
            out.add_(self.bias)
        if self.act == "gelu":
            out.copy_(F.gelu(out, approximate="tanh"))
        elif self.act == "relu":
            out.relu_()


class LayerNormOp(Operator):
    def __init__(self, ctx, name, weight, bias, eps: float = 1e-5):
        super().__init__(ctx, name)
        self.weight, self.bias, self.eps = weight, bias, eps

    def __call__(self, x: Variable) -> Variable:
        out = Variable(self.ctx, self.name + ".out", x.max_shape, x.dtype)
        self._register([x], [out])
        return out

    def run(self, lead):
        from oslo_b200.ops.norm import layer_norm

        x = self.inputs[0].value
        self.outputs[0].value.copy_(layer_norm(x, (x.shape[-1],), self.weight, self.bias, self.eps))


class AddOp(Operator):
    """``out = a + b`` (residual connections)."""

    def __call__(self, a: Variable, b: Variable) -> Variable:
        out = Variable(self.ctx, self.name + ".out", a.max_shape, a.dtype)
        self._register([a, b], [out])
        return out

    def run(self, lead):
        torch.add(self.inputs[0].value, self.inputs[1].value, out=self.outputs[0].value)


class AttentionOp(Operator):
    """Self-attention on a fused QKV variable ``[tokens, 3 * hidden]`` laid out ``[3, heads, head_dim]``; tokens are
    ``batch x seq`` with ``seq`` given per run."""

    def __init__(self, ctx, name, heads: int, causal: bool = False):
        super().__init__(ctx, name)
        self.heads, self.causal = heads, causal

    def __call__(self, qkv: Variable) -> Variable:
        out = Variable(self.ctx, self.name + ".out", (qkv.max_shape[0], qkv.max_shape[1] // 3), qkv.dtype)
        self._register([qkv], [out])
        return out

    def run(self, lead):
        from oslo_b200.ops.attention import qkv_attention

        qkv, out = self.inputs[0].value, self.outputs[0].value
        seq = self.ctx.seq_len
        hd = qkv.shape[-1] // (3 * self.heads)
        y = qkv_attention(qkv.view(lead // seq, seq, qkv.shape[-1]), self.heads, hd, layout="3hd", causal=self.causal)
        out.copy_(y.reshape(lead, -1))


class Context:
    """Graph under construction, then its plan and arena.  ``seq_len`` is read by sequence-aware operators at run time."""

    def __init__(self, device="cpu"):
        self.device = torch.device(device)
        self._variables: List[Variable] = []
        self._nodes: List[Operator] = []
        self._inputs: Dict[str, Variable] = {}
        self.built = False
        self.arena: Optional[torch.Tensor] = None
        self.arena_bytes = self.naive_bytes = 0
        self.seq_len = 1

    # ----------------------------------------------------------------- construction
    def input(self, name: str, max_shape: Sequence[int], dtype=torch.float32) -> Variable:
        v = Variable(self, name, max_shape, dtype, external=True)
        self._inputs[name] = v
        return v

    def build(self) -> "Context":
        """Freeze the graph: lifetimes -> offsets (the planner packs tensors whose lifetimes do not overlap into the same
        bytes) -> one arena allocation."""
        inner = [v for v in self._variables if not v.external]
        sizes = [(v.max_bytes + _ALIGN - 1) // _ALIGN * _ALIGN for v in inner]
        first = [v.first_use for v in inner]
        last = [v.last_use for v in inner]
        offsets, total = plan(sizes, first, last, _ALIGN) if inner else ([], 0)
        if inner and not check(sizes, first, last, offsets):
            raise RuntimeError("memory plan failed its overlap check")
        for v, off in zip(inner, offsets):
            v.offset = off
        self.arena_bytes, self.naive_bytes = total, sum(sizes)
        self.arena = torch.empty(max(total, 1), dtype=torch.uint8, device=self.device)
        self.built = True
        return self

    # ------------------------------------------------------------------------ run
    def run(self, feed: Dict[str, torch.Tensor], outputs: Sequence[Variable], seq_len: Optional[int] = None) -> Tuple[torch.Tensor, ...]:
        """Execute the nodes in construction order.  Every fed tensor's leading dimension must be the same ``lead`` and at
        most the declared maximum.  Returned tensors are views into the arena: copy them before the next run."""
        if not self.built:
            raise RuntimeError("call build() first")
        lead = None
        for name, t in feed.items():
            v = self._inputs[name]
            if t.shape[1:] != v.max_shape[1:] or t.shape[0] > v.max_shape[0]:
                raise ValueError(f"{name}: shape {tuple(t.shape)} does not fit the declared maximum {v.max_shape}")
            lead = t.shape[0] if lead is None else lead
            if t.shape[0] != lead:
                raise ValueError("all inputs must share the leading dimension")
            v.value = t
        missing = set(self._inputs) - set(feed)
        if missing:
            raise ValueError(f"missing inputs {sorted(missing)}")
        if seq_len is not None:
            self.seq_len = seq_len
        for v in self._variables:
            if not v.external:
                v.value = v.view(lead)
        with torch.no_grad():
            for node in self._nodes:
                node.run(lead)
        return tuple(v.value for v in outputs)


def encoder_layer_graph(ctx: Context, x: Variable, layer, name: str) -> Variable:
    """Add one pre-LayerNorm :class:`oslo_b200.lightseq.layers.LSTransformerEncoderLayer` (its parameters are bound, not
    copied) to ``ctx``; returns the layer's output variable."""
    cfg = layer.attn.config
    if not cfg.pre_layer_norm:
        raise ValueError("the graph builder covers pre-LayerNorm layers")
    a, f = layer.attn, layer.ffn
    h = LayerNormOp(ctx, name + ".ln1", a.norm.weight, a.norm.bias, a.norm.eps)(x)
    qkv = LinearOp(ctx, name + ".qkv", a.qkv.weight, a.qkv.bias)(h)
    att = AttentionOp(ctx, name + ".attn", cfg.nhead, causal=a.causal)(qkv)
    proj = LinearOp(ctx, name + ".out", a.out.weight, a.out.bias)(att)
    x1 = AddOp(ctx, name + ".res1")(proj, x)
    h2 = LayerNormOp(ctx, name + ".ln2", f.norm.weight, f.norm.bias, f.norm.eps)(x1)
    up = LinearOp(ctx, name + ".fc1", f.fc1.weight, f.fc1.bias, act=cfg.activation_fn)(h2)
    down = LinearOp(ctx, name + ".fc2", f.fc2.weight, f.fc2.bias)(up)
    return AddOp(ctx, name + ".res2")(down, x1)


__all__ = ["Context", "Variable", "Operator", "LinearOp", "LayerNormOp", "AddOp", "AttentionOp", "encoder_layer_graph"]
