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
    """Symbolic tensor.  ``max_shape[0]`` is the dimension that may shrink at run time: the number of tokens
    (``lead="tokens"``) or of sequences (``lead="batch"``, e.g. pooled outputs); the other dimensions are fixed."""

    def __init__(self, ctx: "Context", name: str, max_shape: Sequence[int], dtype: torch.dtype, external: bool = False,
                 lead: str = "tokens"):
        self.ctx, self.name, self.max_shape, self.dtype, self.external = ctx, name, tuple(int(s) for s in max_shape), dtype, external
        if lead not in ("tokens", "batch"):
            raise ValueError("lead is 'tokens' (batch x seq rows) or 'batch' (one row per sequence)")
        self.lead = lead
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

    def native_record(self, slot):
        """Record of this node for the host executor (``csrc/cpu/graph_exec.cpp``): a dict of the record's fields, with
        tensors / variables given through ``slot(obj)`` (an index into the pointer table), or ``None`` when the executor has
        no such operator (the context then keeps running node by node)."""
        return None


_ACT_CODE = {None: -1, "tanh": 0, "relu": 1, "gelu": 2}
_ROWS = {"tokens": 0, "batch": 1}


def _f64_bits(x: float) -> int:
    import struct

    return struct.unpack("<q", struct.pack("<d", float(x)))[0]


class LinearOp(Operator):
    """``out = act(x @ W^T + b)``; ``act`` in {None, "gelu", "relu"} (GELU rides in the GEMM epilogue on CUDA)."""

    def __init__(self, ctx, name, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, act: Optional[str] = None):
        super().__init__(ctx, name)
        self.weight, self.bias, self.act = weight, bias, act

    def __call__(self, x: Variable) -> Variable:
        out = Variable(self.ctx, self.name + ".out", (x.max_shape[0], self.weight.shape[0]), x.dtype, lead=x.lead)
        self._register([x], [out])
        return out

    def native_record(self, slot):
        if self.act not in _ACT_CODE:
            return None
        return dict(op=1, in0=slot(self.inputs[0]), out=slot(self.outputs[0]), w=slot(self.weight), b=slot(self.bias),
                    rows=_ROWS[self.outputs[0].lead], d0=self.weight.shape[1], d1=self.weight.shape[0], d2=_ACT_CODE[self.act])

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
        out = Variable(self.ctx, self.name + ".out", x.max_shape, x.dtype, lead=x.lead)
        self._register([x], [out])
        return out

    def native_record(self, slot):
        return dict(op=2, in0=slot(self.inputs[0]), out=slot(self.outputs[0]), w=slot(self.weight), b=slot(self.bias),
                    rows=_ROWS[self.outputs[0].lead], d0=self.inputs[0].max_shape[-1], scalar=_f64_bits(self.eps))

    def run(self, lead):
        from oslo_b200.ops.norm import layer_norm

        x = self.inputs[0].value
        self.outputs[0].value.copy_(layer_norm(x, (x.shape[-1],), self.weight, self.bias, self.eps))


class AddOp(Operator):
    """``out = a + b`` (residual connections)."""

    def __call__(self, a: Variable, b: Variable) -> Variable:
        out = Variable(self.ctx, self.name + ".out", a.max_shape, a.dtype, lead=a.lead)
        self._register([a, b], [out])
        return out

    def native_record(self, slot):
        return dict(op=3, in0=slot(self.inputs[0]), in1=slot(self.inputs[1]), out=slot(self.outputs[0]),
                    rows=_ROWS[self.outputs[0].lead], d0=math.prod(self.inputs[0].max_shape[1:]))

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

    def native_record(self, slot):
        hidden = self.inputs[0].max_shape[1] // 3
        return dict(op=4, in0=slot(self.inputs[0]), out=slot(self.outputs[0]), d1=self.heads, d2=hidden // self.heads,
                    flags=1 if self.causal else 0)

    def run(self, lead):
        from oslo_b200.ops.attention import qkv_attention

        qkv, out = self.inputs[0].value, self.outputs[0].value
        seq = self.ctx.seq_len
        hd = qkv.shape[-1] // (3 * self.heads)
        mask = None
        if self.ctx.padding_mask is not None:
            mask = self.ctx.padding_mask.to(torch.float32)[:, None, None, :] * -1e4
        y = qkv_attention(qkv.view(lead // seq, seq, qkv.shape[-1]), self.heads, hd, layout="3hd", causal=self.causal, mask=mask)
        out.copy_(y.reshape(lead, -1))



class EmbeddingOp(Operator):
    """Token ids ``[tokens]`` (int64, row-major ``batch x seq``) -> ``emb[ids] * scale + pos[step + t]`` with padding rows
    zeroed (one kernel on CUDA, ``lightseq/kernels.py:ls_embedding``)."""

    def __init__(self, ctx, name, weight: torch.Tensor, positions: torch.Tensor, padding_idx: int, scale: float):
        super().__init__(ctx, name)
        self.weight, self.positions, self.padding_idx, self.scale = weight, positions, padding_idx, scale

    def __call__(self, ids: Variable) -> Variable:
        out = Variable(self.ctx, self.name + ".out", (ids.max_shape[0], self.weight.shape[1]), self.weight.dtype)
        self._register([ids], [out])
        return out

    def native_record(self, slot):
        pos = self.positions
        if pos.dtype != self.weight.dtype or pos.device != self.weight.device:
            pos = self.positions = pos.to(device=self.weight.device, dtype=self.weight.dtype)
        return dict(op=5, in0=slot(self.inputs[0]), out=slot(self.outputs[0]), w=slot(self.weight), x0=slot(pos),
                    d0=self.weight.shape[1], d2=self.padding_idx, scalar=_f64_bits(self.scale))

    def run(self, lead):
        from .kernels import ls_embedding

        seq = self.ctx.seq_len
        pos = self.positions
        if pos.dtype != self.weight.dtype or pos.device != self.weight.device:
            pos = self.positions = pos.to(device=self.weight.device, dtype=self.weight.dtype)
        y = ls_embedding(self.inputs[0].value.view(lead // seq, seq), self.weight, pos, self.ctx.step, self.padding_idx, self.scale,
                         0.0, False)
        self.outputs[0].value.copy_(y.reshape(lead, -1))


class CachedAttentionOp(Operator):
    """Causal self-attention for incremental decoding.  The keys / values of the tokens of this run are written into two
    persistent buffers ``[max_batch, heads, max_len, head_dim]`` at positions ``[step, step + seq)``; the queries attend
    over positions ``[0, step + seq)``.  A run with ``step = 0`` is the prompt (prefill), later runs feed one token."""

    def __init__(self, ctx, name, heads: int, max_batch: int, max_len: int, head_dim: int, dtype: torch.dtype):
        super().__init__(ctx, name)
        self.heads, self.head_dim, self.max_len = heads, head_dim, max_len
        self.k_name = ctx.persistent(name + ".k_cache", (max_batch, heads, max_len, head_dim), dtype)
        self.v_name = ctx.persistent(name + ".v_cache", (max_batch, heads, max_len, head_dim), dtype)

    def __call__(self, qkv: Variable) -> Variable:
        out = Variable(self.ctx, self.name + ".out", (qkv.max_shape[0], qkv.max_shape[1] // 3), qkv.dtype)
        self._register([qkv], [out])
        return out

    def native_record(self, slot):
        return dict(op=8, in0=slot(self.inputs[0]), out=slot(self.outputs[0]), d1=self.heads, d2=self.head_dim,
                    x0=slot(("buffer", self.k_name)), x1=slot(("buffer", self.v_name)), max_len=self.max_len)

    def run(self, lead):
        ctx = self.ctx
        seq, step = ctx.seq_len, ctx.step
        b = lead // seq
        if step + seq > self.max_len:
            raise ValueError(f"position {step + seq} exceeds the cache length {self.max_len}")
        qkv = self.inputs[0].value.view(b, seq, 3, self.heads, self.head_dim)
        q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        kc, vc = ctx.buffers[self.k_name], ctx.buffers[self.v_name]
        kc[:b, :, step : step + seq].copy_(k)
        vc[:b, :, step : step + seq].copy_(v)
        keys, vals = kc[:b, :, : step + seq], vc[:b, :, : step + seq]
        scores = torch.matmul(q, keys.transpose(-1, -2)).float() * (self.head_dim ** -0.5)
        if seq > 1:  # token i of this run sees cache positions <= step + i
            pos_q = torch.arange(step, step + seq, device=scores.device)[:, None]
            pos_k = torch.arange(step + seq, device=scores.device)[None, :]
            scores = scores.masked_fill(pos_k > pos_q, float("-inf"))
        probs = torch.softmax(scores, dim=-1).to(vals.dtype)
        y = torch.matmul(probs, vals).permute(0, 2, 1, 3).reshape(lead, -1)
        self.outputs[0].value.copy_(y)

    def reorder(self, index: torch.Tensor):
        """Beam search: row ``i`` of the caches becomes the old row ``index[i]``."""
        for name in (self.k_name, self.v_name):
            buf = self.ctx.buffers[name]
            buf[: index.numel()].copy_(buf[index.to(buf.device)].clone())


class CrossAttentionOp(Operator):
    """Decoder -> encoder attention.  ``encode_memory`` projects the encoder output to keys / values once per source batch
    (stored in persistent buffers); each run attends the decoder queries ``[tokens, hidden]`` over them."""

    def __init__(self, ctx, name, heads: int, head_dim: int, kv_weight, kv_bias, max_batch: int, max_src: int, dtype):
        super().__init__(ctx, name)
        self.heads, self.head_dim, self.kv_weight, self.kv_bias = heads, head_dim, kv_weight, kv_bias
        self.k_name = ctx.persistent(name + ".k_mem", (max_batch, heads, max_src, head_dim), dtype)
        self.v_name = ctx.persistent(name + ".v_mem", (max_batch, heads, max_src, head_dim), dtype)
        self.src_len = 0
        self.src_mask: Optional[torch.Tensor] = None

    def __call__(self, q: Variable) -> Variable:
        out = Variable(self.ctx, self.name + ".out", q.max_shape, q.dtype)
        self._register([q], [out])
        return out

    def encode_memory(self, encoder_out: torch.Tensor, padding_mask: Optional[torch.Tensor] = None):
        b, s, _ = encoder_out.shape
        kv = F.linear(encoder_out, self.kv_weight, self.kv_bias).view(b, s, 2, self.heads, self.head_dim)
        self.ctx.buffers[self.k_name][:b, :, :s].copy_(kv[:, :, 0].permute(0, 2, 1, 3))
        self.ctx.buffers[self.v_name][:b, :, :s].copy_(kv[:, :, 1].permute(0, 2, 1, 3))
        self.src_len, self.src_mask = s, padding_mask

    def run(self, lead):
        seq = self.ctx.seq_len
        b = lead // seq
        q = self.inputs[0].value.view(b, seq, self.heads, self.head_dim).permute(0, 2, 1, 3)
        k = self.ctx.buffers[self.k_name][:b, :, : self.src_len]
        v = self.ctx.buffers[self.v_name][:b, :, : self.src_len]
        scores = torch.matmul(q, k.transpose(-1, -2)).float() * (self.head_dim ** -0.5)
        if self.src_mask is not None:
            scores = scores + self.src_mask.to(torch.float32)[:b, None, None, :] * -1e4
        probs = torch.softmax(scores, dim=-1).to(v.dtype)
        self.outputs[0].value.copy_(torch.matmul(probs, v).permute(0, 2, 1, 3).reshape(lead, -1))

    def reorder(self, index: torch.Tensor):
        for name in (self.k_name, self.v_name):
            buf = self.ctx.buffers[name]
            buf[: index.numel()].copy_(buf[index.to(buf.device)].clone())
        if self.src_mask is not None:
            self.src_mask = self.src_mask[index.to(self.src_mask.device)]


class SelectTokenOp(Operator):
    """One row per sequence: the first (``which=0``, BERT pooling) or the last (``which=-1``, next-token logits) token."""

    def __init__(self, ctx, name, which: int = 0):
        super().__init__(ctx, name)
        self.which = which

    def __call__(self, x: Variable) -> Variable:
        out = Variable(self.ctx, self.name + ".out", x.max_shape, x.dtype, lead="batch")
        self._register([x], [out])
        return out

    def native_record(self, slot):
        return dict(op=6, in0=slot(self.inputs[0]), out=slot(self.outputs[0]), rows=1, d0=self.inputs[0].max_shape[-1], d2=self.which)

    def run(self, lead):
        seq = self.ctx.seq_len
        x = self.inputs[0].value.view(lead // seq, seq, -1)
        self.outputs[0].value.copy_(x[:, self.which])


class ActivationOp(Operator):
    """Element-wise ``tanh`` / ``relu`` / ``gelu``; keeps the lead kind of its input."""

    _FN = {"tanh": torch.tanh, "relu": torch.relu, "gelu": lambda x: F.gelu(x, approximate="tanh")}

    def __init__(self, ctx, name, kind: str):
        super().__init__(ctx, name)
        self.kind = kind

    def __call__(self, x: Variable) -> Variable:
        out = Variable(self.ctx, self.name + ".out", x.max_shape, x.dtype, lead=x.lead)
        self._register([x], [out])
        return out

    def native_record(self, slot):
        return dict(op=7, in0=slot(self.inputs[0]), out=slot(self.outputs[0]), rows=_ROWS[self.outputs[0].lead],
                    d0=math.prod(self.inputs[0].max_shape[1:]), d2=_ACT_CODE[self.kind])

    def run(self, lead):
        self.outputs[0].value.copy_(self._FN[self.kind](self.inputs[0].value))


class CRFDecodeOp(Operator):
    """Viterbi decoding of emissions ``[tokens, tags]`` with a linear-chain CRF's transition scores; writes the best tag
    of every token (``[tokens]`` int64; padding positions get -1)."""

    def __init__(self, ctx, name, crf):
        super().__init__(ctx, name)
        self.crf = crf

    def __call__(self, emissions: Variable) -> Variable:
        out = Variable(self.ctx, self.name + ".out", (emissions.max_shape[0],), torch.int64)
        self._register([emissions], [out])
        return out

    def run(self, lead):
        seq = self.ctx.seq_len
        em = self.inputs[0].value.view(lead // seq, seq, -1).float()
        mask = None if self.ctx.padding_mask is None else ~self.ctx.padding_mask
        paths = self.crf.decode(em, mask)
        out = self.outputs[0].value.view(lead // seq, seq)
        out.fill_(-1)
        for i, path in enumerate(paths):
            out[i, : len(path)] = torch.as_tensor(path, dtype=torch.int64, device=out.device)


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
        self.step = 0  # position of the first token of this run (incremental decoding)
        self.padding_mask: Optional[torch.Tensor] = None  # [batch, seq] bool, True at padding; None = no padding
        self._persistent: List[Tuple[str, Tuple[int, ...], torch.dtype]] = []
        self.buffers: Dict[str, torch.Tensor] = {}

    # ----------------------------------------------------------------- construction
    def input(self, name: str, max_shape: Sequence[int], dtype=torch.float32, lead: str = "tokens") -> Variable:
        v = Variable(self, name, max_shape, dtype, external=True, lead=lead)
        self._inputs[name] = v
        return v

    def persistent(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> str:
        """Declare a buffer that keeps its contents between runs (key / value caches): allocated once in ``build()``,
        outside the arena, read through ``ctx.buffers[name]``."""
        if self.built:
            raise RuntimeError("the graph is frozen after build()")
        self._persistent.append((name, tuple(int(s) for s in shape), dtype))
        return name

    @property
    def persistent_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.buffers.values())

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
        for name, shape, dtype in self._persistent:
            self.buffers[name] = torch.zeros(shape, dtype=dtype, device=self.device)
        self.built = True
        return self

    # ---------------------------------------------------------------- native program
    _FIELDS = ("op", "in0", "in1", "out", "w", "b", "rows", "d0", "d1", "d2", "flags", "scalar", "x0", "x1", "max_len", "reserved")

    def compile_native(self) -> bool:
        """Translate the graph into a program for the host executor (``csrc/cpu/graph_exec.cpp``): afterwards a run is
        one native call instead of one Python dispatch per node.  Possible when the graph lives on the CPU in fp32 and every
        node has a native operator; returns whether it was (the node-by-node path stays available either way)."""
        if not self.built:
            raise RuntimeError("call build() first")
        self._native = None
        if self.device.type != "cpu":
            return False
        if any(v.dtype not in (torch.float32, torch.int64) for v in self._variables):
            return False
        items: List[object] = []
        index: Dict[object, int] = {}

        def slot(obj) -> int:
            if obj is None:
                return -1
            key = obj if isinstance(obj, tuple) else id(obj)
            if key not in index:
                if torch.is_tensor(obj) and (obj.dtype != torch.float32 or not obj.is_contiguous() or obj.device.type != "cpu"):
                    raise TypeError("native programs take contiguous fp32 host tensors")
                index[key] = len(items)
                items.append(obj)
            return index[key]

        records = []
        try:
            for node in self._nodes:
                rec = node.native_record(slot)
                if rec is None:
                    return False
                row = [-1 if f in ("in0", "in1", "out", "w", "b", "x0", "x1") else 0 for f in self._FIELDS]
                for k, v in rec.items():
                    row[self._FIELDS.index(k)] = int(v)
                records.append(row)
        except TypeError:
            return False
        import ctypes

        from oslo_b200.ops import _lib

        lib = _lib.cpu_lib()
        if lib.oslo_cpu_graph_record_size() != len(self._FIELDS):
            return False
        lib.oslo_cpu_graph_run.restype = ctypes.c_int
        self._native = {"lib": lib, "prog": torch.tensor(records, dtype=torch.int64).contiguous(), "items": items,
                        "ptrs": (ctypes.c_void_p * max(len(items), 1))()}
        return True

    def _run_native(self, lead: int) -> None:
        import ctypes

        nat = self._native
        ptrs = nat["ptrs"]
        for i, obj in enumerate(nat["items"]):
            if isinstance(obj, Variable):
                t = obj.value
                if not t.is_contiguous():
                    t = obj.value = t.contiguous()
            elif isinstance(obj, tuple):
                t = self.buffers[obj[1]]
            else:
                t = obj
            ptrs[i] = t.data_ptr()
        pad = self.padding_mask
        pad_t = None
        if pad is not None:
            pad_t = pad.to(torch.uint8).contiguous()
        rc = nat["lib"].oslo_cpu_graph_run(
            ctypes.c_void_p(nat["prog"].data_ptr()), ctypes.c_int(nat["prog"].shape[0]), ptrs, ctypes.c_longlong(lead),
            ctypes.c_longlong(self.seq_len), ctypes.c_longlong(self.step), ctypes.c_void_p(pad_t.data_ptr() if pad_t is not None else None))
        if rc != 0:
            node = self._nodes[-rc - 1].name if -len(self._nodes) <= rc < 0 else "?"
            raise RuntimeError(f"the host graph executor stopped at node {node!r} (code {rc})")

    # ------------------------------------------------------------------------ run
    def run(self, feed: Dict[str, torch.Tensor], outputs: Sequence[Variable], seq_len: Optional[int] = None, step: int = 0,
            padding_mask: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, ...]:
        """Execute the nodes in construction order.  Every fed token-major tensor's leading dimension must be the same
        ``lead`` (a multiple of ``seq_len``) and at most the declared maximum.  ``step``: position of the first token
        (incremental decoding over the persistent caches); ``padding_mask``: ``[batch, seq]``, True at padding.
        Returned tensors are views into the arena: copy them before the next run."""
        if not self.built:
            raise RuntimeError("call build() first")
        lead = None
        for name, t in feed.items():
            v = self._inputs[name]
            if t.shape[1:] != v.max_shape[1:] or t.shape[0] > v.max_shape[0]:
                raise ValueError(f"{name}: shape {tuple(t.shape)} does not fit the declared maximum {v.max_shape}")
            if v.lead == "tokens":
                lead = t.shape[0] if lead is None else lead
                if t.shape[0] != lead:
                    raise ValueError("all token-major inputs must share the leading dimension")
            v.value = t
        missing = set(self._inputs) - set(feed)
        if missing:
            raise ValueError(f"missing inputs {sorted(missing)}")
        if seq_len is not None:
            self.seq_len = seq_len
        if lead is None:
            raise ValueError("no token-major input was fed")
        if lead % self.seq_len:
            raise ValueError(f"{lead} rows are not a multiple of seq_len {self.seq_len}")
        batch = lead // self.seq_len
        self.step, self.padding_mask = int(step), padding_mask
        for v in self._variables:
            if not v.external:
                v.value = v.view(lead if v.lead == "tokens" else batch)
        with torch.no_grad():
            if getattr(self, "_native", None) is not None:
                self._run_native(lead)
            else:
                for node in self._nodes:
                    node.run(lead)
        return tuple(v.value for v in outputs)


def _attention_block(ctx: Context, x: Variable, a, name: str, attn_op: Operator) -> Variable:
    """LayerNorm placement, fused QKV projection, ``attn_op``, output projection and residual of one attention block."""
    pre = a.config.pre_layer_norm
    h = LayerNormOp(ctx, name + ".ln", a.norm.weight, a.norm.bias, a.norm.eps)(x) if pre else x
    qkv = LinearOp(ctx, name + ".qkv", a.qkv.weight, a.qkv.bias)(h)
    proj = LinearOp(ctx, name + ".out", a.out.weight, a.out.bias)(attn_op(qkv))
    y = AddOp(ctx, name + ".res")(proj, x)
    return y if pre else LayerNormOp(ctx, name + ".ln", a.norm.weight, a.norm.bias, a.norm.eps)(y)


def _ffn_block(ctx: Context, x: Variable, f, name: str) -> Variable:
    pre = f.config.pre_layer_norm
    h = LayerNormOp(ctx, name + ".ln", f.norm.weight, f.norm.bias, f.norm.eps)(x) if pre else x
    up = LinearOp(ctx, name + ".fc1", f.fc1.weight, f.fc1.bias, act=f.config.activation_fn)(h)
    down = LinearOp(ctx, name + ".fc2", f.fc2.weight, f.fc2.bias)(up)
    y = AddOp(ctx, name + ".res")(down, x)
    return y if pre else LayerNormOp(ctx, name + ".ln", f.norm.weight, f.norm.bias, f.norm.eps)(y)


def encoder_layer_graph(ctx: Context, x: Variable, layer, name: str, cache: Optional[Tuple[int, int]] = None) -> Variable:
    """Add one :class:`oslo_b200.lightseq.layers.LSTransformerEncoderLayer` / ``LSGptEncoderLayer`` (pre- or
    post-LayerNorm; its parameters are bound, not copied) to ``ctx``; returns the layer's output variable.  ``cache =
    (max_batch, max_len)`` builds the causal attention over a persistent key / value cache (incremental decoding)."""
    a = layer.attn
    cfg = a.config
    if cache is not None:
        op = CachedAttentionOp(ctx, name + ".attn", cfg.nhead, cache[0], cache[1], a.head_dim, a.qkv.weight.dtype)
    else:
        op = AttentionOp(ctx, name + ".attn", cfg.nhead, causal=a.causal)
    return _ffn_block(ctx, _attention_block(ctx, x, a, name + ".self", op), layer.ffn, name + ".ffn")


def decoder_layer_graph(ctx: Context, x: Variable, layer, name: str, max_batch: int, max_len: int, max_src: int):
    """One :class:`oslo_b200.lightseq.layers.LSTransformerDecoderLayer`: cached causal self-attention, attention over the
    encoder memory, feed-forward.  Returns ``(output variable, cross-attention operator)``; the caller feeds the encoder
    output to the operator's ``encode_memory`` once per source batch."""
    a, c = layer.self_attn, layer.cross_attn
    cfg = a.config
    dtype = a.qkv.weight.dtype
    self_op = CachedAttentionOp(ctx, name + ".self.attn", cfg.nhead, max_batch, max_len, a.head_dim, dtype)
    x = _attention_block(ctx, x, a, name + ".self", self_op)
    pre = cfg.pre_layer_norm
    h = LayerNormOp(ctx, name + ".cross.ln", c.norm.weight, c.norm.bias, c.norm.eps)(x) if pre else x
    q = LinearOp(ctx, name + ".cross.q", c.q.weight, c.q.bias)(h)
    cross = CrossAttentionOp(ctx, name + ".cross.attn", cfg.nhead, c.head_dim, c.kv.weight, c.kv.bias, max_batch, max_src, dtype)
    proj = LinearOp(ctx, name + ".cross.out", c.out.weight, c.out.bias)(cross(q))
    y = AddOp(ctx, name + ".cross.res")(proj, x)
    if not pre:
        y = LayerNormOp(ctx, name + ".cross.ln", c.norm.weight, c.norm.bias, c.norm.eps)(y)
    return _ffn_block(ctx, y, layer.ffn, name + ".ffn"), cross


__all__ = ["Context", "Variable", "Operator", "LinearOp", "LayerNormOp", "AddOp", "AttentionOp", "EmbeddingOp", "CachedAttentionOp",
           "CrossAttentionOp", "SelectTokenOp", "ActivationOp", "CRFDecodeOp", "encoder_layer_graph", "decoder_layer_graph"]
