"""Quantiser module and quantised layers.

Parity: oslo/lightseq2/training/pytorch_quantization/nn/modules/{tensor_quantizer,clip,quant_linear,quant_conv,quant_pooling,
quant_instancenorm,quant_bert,_utils}.py.  :class:`TensorQuantizer` has three switches, independent of one another:
*calibrate* (feed inputs to its calibrator), *clip* (clamp to a learned range without rounding: the first stage of
clip-then-quantise training) and *quantise* (fake or real quantisation with the straight-through gradient).  The quantised
layers quantise their input and their weight and then run the ordinary float op, which is what int8 inference computes up to
accumulation order.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import calib
from .tensor_quant import (QUANT_DESC_8BIT_CONV_WEIGHT_PER_CHANNEL, QUANT_DESC_8BIT_CONVTRANSPOSE_WEIGHT_PER_CHANNEL,
                           QUANT_DESC_8BIT_LINEAR_WEIGHT_PER_ROW, QUANT_DESC_8BIT_PER_TENSOR, QuantDescriptor, fake_tensor_quant,
                           reduce_amax, tensor_quant)


class Clip(nn.Module):
    """``clamp(x, lo, hi)`` with optionally learned bounds; the bounds receive the gradient of the clipped elements."""

    def __init__(self, clip_value_min, clip_value_max, learn_min: bool = False, learn_max: bool = False):
        super().__init__()
        lo, hi = torch.as_tensor(clip_value_min, dtype=torch.float32), torch.as_tensor(clip_value_max, dtype=torch.float32)
        self.clip_value_min = nn.Parameter(lo) if learn_min else lo
        self.clip_value_max = nn.Parameter(hi) if learn_max else hi
        if not learn_min:
            self.register_buffer("_lo", lo, persistent=False)
        if not learn_max:
            self.register_buffer("_hi", hi, persistent=False)

    def forward(self, x):
        lo = self.clip_value_min if isinstance(self.clip_value_min, nn.Parameter) else self._lo
        hi = self.clip_value_max if isinstance(self.clip_value_max, nn.Parameter) else self._hi
        return torch.minimum(torch.maximum(x, lo.to(x.dtype)), hi.to(x.dtype))


class TensorQuantizer(nn.Module):
    """Quantiser of one tensor, configured by a :class:`QuantDescriptor`.

    With no ``amax`` (never calibrated, none given) every call uses the maximum of its own input ("dynamic" quantisation).
    For backward compatibility the first positional argument may be ``num_bits`` with ``axis`` as keyword."""

    def __init__(self, quant_desc=None, disabled: bool = False, if_quant: bool = True, if_clip: bool = False, if_calib: bool = False,
                 axis=None, **desc_kwargs):
        super().__init__()
        if isinstance(quant_desc, int):
            quant_desc = QuantDescriptor(num_bits=quant_desc, axis=axis, **desc_kwargs)
        elif quant_desc is None:
            quant_desc = QuantDescriptor(axis=axis, **desc_kwargs)
        d = quant_desc
        self._num_bits, self._unsigned, self._narrow_range, self._fake_quant = d.num_bits, d.unsigned, d.narrow_range, d.fake_quant
        self._axis, self._scale_amax, self._learn_amax = d.axis, d.scale_amax, d.learn_amax
        self._disabled, self._if_quant, self._if_clip, self._if_calib = disabled, if_quant, False, if_calib
        self._scale: Optional[torch.Tensor] = None
        if d.amax is not None:
            amax = torch.tensor(d.amax, dtype=torch.float32)
            if d.learn_amax:
                self._amax = nn.Parameter(amax)
            else:
                self.register_buffer("_amax", amax)
        if d.calib_method == "histogram":
            self._calibrator = calib.HistogramCalibrator(d.num_bits, d.axis, d.unsigned)
        else:
            self._calibrator = calib.MaxCalibrator(d.num_bits, d.axis, d.unsigned)
        if if_clip:
            self.enable_clip()

    # ------------------------------------------------------------- properties
    num_bits = property(lambda self: self._num_bits)
    unsigned = property(lambda self: self._unsigned)
    narrow_range = property(lambda self: self._narrow_range)
    fake_quant = property(lambda self: self._fake_quant)
    axis = property(lambda self: self._axis)
    scale = property(lambda self: self._scale)

    @property
    def amax(self) -> Optional[torch.Tensor]:
        return getattr(self, "_amax", None)

    @amax.setter
    def amax(self, value):
        if value is None:
            raise ValueError("amax cannot be reset to None; build a new quantiser")
        value = torch.as_tensor(value, dtype=torch.float32).detach().clone()
        cur = getattr(self, "_amax", None)
        if cur is None:
            self.register_buffer("_amax", value)
        elif cur.shape == value.shape:
            cur.data.copy_(value.to(cur.device))
        elif isinstance(cur, nn.Parameter):
            raise ValueError(f"learned amax has shape {tuple(cur.shape)}, not {tuple(value.shape)}")
        else:
            self._amax = value.to(cur.device)

    @property
    def step_size(self) -> Optional[torch.Tensor]:
        if self.amax is None:
            return None
        return self.amax / (2.0 ** (self._num_bits - 1 + int(self._unsigned)) - 1.0)

    # ---------------------------------------------------------------- switches
    def disable(self):
        self._disabled = True

    def enable(self):
        self._disabled = False

    def enable_quant(self):
        self._if_quant = True

    def disable_quant(self):
        self._if_quant = False

    def enable_calib(self):
        if self._calibrator is None:
            raise RuntimeError("this quantiser has no calibrator")
        self._if_calib = True

    def disable_calib(self):
        self._if_calib = False

    def enable_clip(self):
        """Clamp to ``[-amax, amax]`` (``[0, amax]`` when unsigned) with ``amax`` trained; needs ``amax`` to exist."""
        if self.amax is None:
            raise ValueError("clipping needs an amax (give one in the descriptor or calibrate first)")
        if not isinstance(self._amax, nn.Parameter):
            self.init_learn_amax()
        self._if_clip = True

    def disable_clip(self):
        self._if_clip = False

    def init_learn_amax(self):
        """Turn the calibrated ``amax`` buffer into a trained parameter."""
        if self.amax is None:
            raise ValueError("no amax to learn from")
        if not isinstance(self._amax, nn.Parameter):
            value = self._amax.detach().clone()
            del self._amax
            self._amax = nn.Parameter(value)
        self._learn_amax = True

    def load_calib_amax(self, *args, strict: bool = True, **kwargs):
        """Take ``amax`` from the calibrator (arguments go to its ``compute_amax``).  ``strict=False`` tolerates a
        calibrator that has seen no data."""
        value = self._calibrator.compute_amax(*args, **kwargs)
        if value is None:
            if strict:
                raise RuntimeError("the calibrator has collected no data; run a calibration pass first")
            return
        self.amax = value

    # ----------------------------------------------------------------- forward
    def _current_amax(self, x):
        amax = self.amax
        if amax is None:
            amax = reduce_amax(x, self._axis)
        elif self._axis is not None and amax.dim() != x.dim() and amax.numel() > 1:
            ax = (self._axis if isinstance(self._axis, int) else self._axis[0]) % x.dim()
            shape = [1] * x.dim()
            shape[ax] = -1
            amax = amax.view(shape)
        if self._scale_amax:
            amax = amax * self._scale_amax
        return amax

    def forward(self, x):
        if self._disabled:
            return x
        if self._if_calib:
            self._calibrator.collect(x)
        out = x
        if self._if_clip:
            a = self._current_amax(x).to(x.dtype)
            lo = torch.zeros_like(a) if self._unsigned else -a
            out = torch.minimum(torch.maximum(out, lo), a)
        if self._if_quant:
            amax = self._current_amax(out)
            if self._learn_amax and isinstance(getattr(self, "_amax", None), nn.Parameter) and not self._if_clip:
                # trained step size: clamp with a differentiable bound, then round with the straight-through gradient
                a = amax.to(out.dtype)
                lo = torch.zeros_like(a) if self._unsigned else -a
                out = torch.minimum(torch.maximum(out, lo), a)
            if self._fake_quant:
                out = fake_tensor_quant(out, amax.detach(), self._num_bits, self._unsigned, self._narrow_range)
            else:
                out, self._scale = tensor_quant(out, amax.detach(), self._num_bits, self._unsigned, self._narrow_range)
        return out

    def extra_repr(self) -> str:
        if self._disabled:
            return "disabled"
        amax = self.amax
        if amax is None:
            a = "dynamic"
        elif amax.numel() == 1:
            a = f"{float(amax):.4f}"
        else:
            a = f"[{float(amax.min()):.4f}, {float(amax.max()):.4f}]({amax.numel()})"
        flags = "".join(c for c, on in (("Q", self._if_quant), ("C", self._if_clip), ("K", self._if_calib)) if on)
        return (f"{'u' if self._unsigned else ''}int{self._num_bits}{' narrow' if self._narrow_range else ''} "
                f"{'fake' if self._fake_quant else 'real'} axis={self._axis} amax={a} [{flags}]")

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        """An ``_amax`` in the checkpoint creates (or reshapes) the buffer, so calibrated models reload into fresh ones."""
        key = prefix + "_amax"
        if key in state_dict:
            value = state_dict[key]
            cur = getattr(self, "_amax", None)
            if cur is None:
                self.register_buffer("_amax", torch.empty_like(value, dtype=torch.float32))
            elif cur.shape != value.shape and not isinstance(cur, nn.Parameter):
                self._amax = torch.empty_like(value, dtype=torch.float32)
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)


def _each_quantizer(model: nn.Module):
    return (m for m in model.modules() if isinstance(m, TensorQuantizer))


def enable_quant(model):
    for q in _each_quantizer(model):
        q.enable_quant()


def disable_quant(model):
    for q in _each_quantizer(model):
        q.disable_quant()


def qat_mode(model):
    """Quantisation-aware training: clip and quantise, no statistics."""
    for q in _each_quantizer(model):
        q.enable()
        q.enable_quant()
        q.disable_calib()


def ptq_mode(model):
    """Post-training quantisation: quantise with the calibrated ranges, nothing trained."""
    for q in _each_quantizer(model):
        q.enable()
        q.enable_quant()
        q.disable_clip()
        q.disable_calib()


def collect_stats(model: nn.Module, batches, num_batches: Optional[int] = None, forward=None) -> int:
    """Calibration pass: quantisation off, calibrators on, ``model(**batch)`` (or ``forward(model, batch)``) under
    ``no_grad`` for up to ``num_batches`` batches.  Returns how many were run."""
    for q in _each_quantizer(model):
        q.disable_quant()
        q.enable_calib()
    done = 0
    was_training = model.training
    model.eval()
    with torch.no_grad():
        for batch in batches:
            if num_batches is not None and done >= num_batches:
                break
            if forward is not None:
                forward(model, batch)
            elif isinstance(batch, dict):
                model(**batch)
            elif isinstance(batch, (tuple, list)):
                model(*batch)
            else:
                model(batch)
            done += 1
    model.train(was_training)
    for q in _each_quantizer(model):
        q.enable_quant()
        q.disable_calib()
    return done


def compute_amax(model: nn.Module, method: str = "max", strict: bool = False, **kwargs) -> None:
    """Load every quantiser's ``amax`` from its calibrator: ``"max"`` for max calibrators; ``"percentile"`` / ``"mse"`` /
    ``"entropy"`` (with their keyword arguments) for histogram calibrators."""
    for q in _each_quantizer(model):
        if isinstance(q._calibrator, calib.MaxCalibrator):
            q.load_calib_amax(strict=strict)
        else:
            q.load_calib_amax(method if method != "max" else "percentile", strict=strict, **kwargs)


class QuantMixin:
    """Input + weight quantisers built from class-level default descriptors (overridable per instance)."""

    default_quant_desc_input = QUANT_DESC_8BIT_PER_TENSOR
    default_quant_desc_weight = QUANT_DESC_8BIT_PER_TENSOR

    @classmethod
    def set_default_quant_desc_input(cls, desc: QuantDescriptor):
        cls.default_quant_desc_input = desc

    @classmethod
    def set_default_quant_desc_weight(cls, desc: QuantDescriptor):
        cls.default_quant_desc_weight = desc

    def init_quantizer(self, quant_desc_input=None, quant_desc_weight=None, num_bits: Optional[int] = None):
        di = quant_desc_input or type(self).default_quant_desc_input
        dw = quant_desc_weight or type(self).default_quant_desc_weight
        if num_bits is not None and num_bits != 8:
            di = QuantDescriptor(**{**_fields(di), "num_bits": num_bits})
            dw = QuantDescriptor(**{**_fields(dw), "num_bits": num_bits})
        self.input_quantizer = TensorQuantizer(di)
        self.weight_quantizer = TensorQuantizer(dw)


class QuantInputMixin:
    """Input quantiser only (pooling, normalisation)."""

    default_quant_desc_input = QUANT_DESC_8BIT_PER_TENSOR

    @classmethod
    def set_default_quant_desc_input(cls, desc: QuantDescriptor):
        cls.default_quant_desc_input = desc

    def init_quantizer(self, quant_desc_input=None):
        self.input_quantizer = TensorQuantizer(quant_desc_input or type(self).default_quant_desc_input)


def _fields(d: QuantDescriptor):
    return {k: getattr(d, k) for k in QuantDescriptor._FIELDS}


def pop_quant_desc_in_kwargs(cls, input_only: bool = False, **kwargs):
    """Split ``quant_desc_input`` / ``quant_desc_weight`` out of a constructor's keyword arguments."""
    di = kwargs.pop("quant_desc_input", cls.default_quant_desc_input)
    if input_only:
        if kwargs:
            raise TypeError(f"unexpected keyword arguments {sorted(kwargs)}")
        return di
    dw = kwargs.pop("quant_desc_weight", cls.default_quant_desc_weight)
    if kwargs:
        raise TypeError(f"unexpected keyword arguments {sorted(kwargs)}")
    return di, dw


class QuantLinear(nn.Linear, QuantMixin):
    """Linear layer with a per-tensor input quantiser and a per-output-row weight quantiser."""

    default_quant_desc_weight = QUANT_DESC_8BIT_LINEAR_WEIGHT_PER_ROW

    def __init__(self, in_features, out_features, bias=True, num_bits: int = 8, **kwargs):
        super().__init__(in_features, out_features, bias)
        di, dw = pop_quant_desc_in_kwargs(type(self), **kwargs)
        self.init_quantizer(di, dw, num_bits)

    def forward(self, x):
        return F.linear(self.input_quantizer(x), self.weight_quantizer(self.weight), self.bias)


Linear = QuantLinear


class _QuantConvNd(QuantMixin):
    default_quant_desc_weight = QUANT_DESC_8BIT_CONV_WEIGHT_PER_CHANNEL

    def _quant(self, x):
        return self.input_quantizer(x), self.weight_quantizer(self.weight)


def _make_conv(base, name, transposed=False):
    class _Q(base, _QuantConvNd):
        default_quant_desc_weight = (QUANT_DESC_8BIT_CONVTRANSPOSE_WEIGHT_PER_CHANNEL if transposed
                                     else QUANT_DESC_8BIT_CONV_WEIGHT_PER_CHANNEL)

        def __init__(self, *args, **kwargs):
            qd = {k: kwargs.pop(k) for k in ("quant_desc_input", "quant_desc_weight") if k in kwargs}
            base.__init__(self, *args, **kwargs)
            di, dw = pop_quant_desc_in_kwargs(type(self), **qd)
            self.init_quantizer(di, dw)

        def forward(self, x, output_size=None):
            xq, wq = self._quant(x)
            if transposed:
                dims = self.weight.dim() - 2
                pad = self._output_padding(x, output_size, self.stride, self.padding, self.kernel_size, dims, self.dilation)
                fn = (F.conv_transpose1d, F.conv_transpose2d, F.conv_transpose3d)[dims - 1]
                return fn(xq, wq, self.bias, self.stride, self.padding, pad, self.groups, self.dilation)
            return self._conv_forward(xq, wq, self.bias)

    _Q.__name__ = _Q.__qualname__ = name
    _Q.__doc__ = f"``torch.nn.{base.__name__}`` with quantised input and per-channel quantised weight."
    return _Q


QuantConv1d = _make_conv(nn.Conv1d, "QuantConv1d")
QuantConv2d = _make_conv(nn.Conv2d, "QuantConv2d")
QuantConv3d = _make_conv(nn.Conv3d, "QuantConv3d")
QuantConvTranspose1d = _make_conv(nn.ConvTranspose1d, "QuantConvTranspose1d", True)
QuantConvTranspose2d = _make_conv(nn.ConvTranspose2d, "QuantConvTranspose2d", True)
QuantConvTranspose3d = _make_conv(nn.ConvTranspose3d, "QuantConvTranspose3d", True)


def _make_input_only(base, name):
    class _Q(base, QuantInputMixin):
        def __init__(self, *args, **kwargs):
            qd = {k: kwargs.pop(k) for k in ("quant_desc_input",) if k in kwargs}
            base.__init__(self, *args, **kwargs)
            self.init_quantizer(pop_quant_desc_in_kwargs(type(self), True, **qd))

        def forward(self, x):
            return base.forward(self, self.input_quantizer(x))

    _Q.__name__ = _Q.__qualname__ = name
    _Q.__doc__ = f"``torch.nn.{base.__name__}`` on a quantised input."
    return _Q


QuantMaxPool1d = _make_input_only(nn.MaxPool1d, "QuantMaxPool1d")
QuantMaxPool2d = _make_input_only(nn.MaxPool2d, "QuantMaxPool2d")
QuantMaxPool3d = _make_input_only(nn.MaxPool3d, "QuantMaxPool3d")
QuantAvgPool1d = _make_input_only(nn.AvgPool1d, "QuantAvgPool1d")
QuantAvgPool2d = _make_input_only(nn.AvgPool2d, "QuantAvgPool2d")
QuantAvgPool3d = _make_input_only(nn.AvgPool3d, "QuantAvgPool3d")
QuantAdaptiveAvgPool1d = _make_input_only(nn.AdaptiveAvgPool1d, "QuantAdaptiveAvgPool1d")
QuantAdaptiveAvgPool2d = _make_input_only(nn.AdaptiveAvgPool2d, "QuantAdaptiveAvgPool2d")
QuantAdaptiveAvgPool3d = _make_input_only(nn.AdaptiveAvgPool3d, "QuantAdaptiveAvgPool3d")
QuantInstanceNorm1d = _make_input_only(nn.InstanceNorm1d, "QuantInstanceNorm1d")
QuantInstanceNorm2d = _make_input_only(nn.InstanceNorm2d, "QuantInstanceNorm2d")
QuantInstanceNorm3d = _make_input_only(nn.InstanceNorm3d, "QuantInstanceNorm3d")


class QuantEmbedding(nn.Embedding, QuantMixin):
    """Embedding table quantised per tensor (the looked-up rows are what int8 inference stores)."""

    def __init__(self, *args, **kwargs):
        qd = {k: kwargs.pop(k) for k in ("quant_desc_weight",) if k in kwargs}
        super().__init__(*args, **kwargs)
        self.weight_quantizer = TensorQuantizer(qd.get("quant_desc_weight", QUANT_DESC_8BIT_PER_TENSOR))

    def forward(self, ids):
        return F.embedding(ids, self.weight_quantizer(self.weight), self.padding_idx, self.max_norm, self.norm_type,
                           self.scale_grad_by_freq, self.sparse)


class QuantMatmul(nn.Module):
    """``a @ b`` with both operands quantised: the two batched products of self-attention in a quantised encoder
    (the counterpart of the quantisers the reference adds inside its BERT self-attention)."""

    def __init__(self, quant_desc_a: Optional[QuantDescriptor] = None, quant_desc_b: Optional[QuantDescriptor] = None):
        super().__init__()
        self.a_quantizer = TensorQuantizer(quant_desc_a or QUANT_DESC_8BIT_PER_TENSOR)
        self.b_quantizer = TensorQuantizer(quant_desc_b or QUANT_DESC_8BIT_PER_TENSOR)

    def forward(self, a, b):
        return torch.matmul(self.a_quantizer(a), self.b_quantizer(b))


class QuantSelfAttention(nn.Module):
    """Multi-head self-attention with every GEMM operand quantised: Q / K / V / output projections are
    :class:`QuantLinear`; scores and context go through :class:`QuantMatmul` (softmax output quantised unsigned)."""

    def __init__(self, hidden_size: int, num_heads: int, dropout: float = 0.0):
        super().__init__()
        if hidden_size % num_heads:
            raise ValueError("hidden_size must be a multiple of num_heads")
        self.h, self.d = num_heads, hidden_size // num_heads
        self.query, self.key, self.value = (QuantLinear(hidden_size, hidden_size) for _ in range(3))
        self.out = QuantLinear(hidden_size, hidden_size)
        self.scores = QuantMatmul()
        self.context = QuantMatmul(QuantDescriptor(num_bits=8, unsigned=True))
        self.dropout = nn.Dropout(dropout)

    def forward(self, x, attention_mask=None):
        b, s, _ = x.shape
        split = lambda t: t.view(b, s, self.h, self.d).transpose(1, 2)
        q, k, v = split(self.query(x)), split(self.key(x)), split(self.value(x))
        att = self.scores(q, k.transpose(-1, -2)) / self.d ** 0.5
        if attention_mask is not None:
            att = att + attention_mask
        p = self.dropout(torch.softmax(att, dim=-1))
        ctx = self.context(p, v).transpose(1, 2).reshape(b, s, self.h * self.d)
        return self.out(ctx)


__all__ = [n for n in dir() if n.startswith("Quant") or n in (
    "Clip", "TensorQuantizer", "Linear", "enable_quant", "disable_quant", "qat_mode", "ptq_mode", "collect_stats", "compute_amax",
    "pop_quant_desc_in_kwargs")]
