"""Quantisation descriptors and the (fake) quantisation functions with straight-through gradients.

Parity: oslo/lightseq2/training/pytorch_quantization/tensor_quant.py (``ScaledQuantDescriptor``, ``TensorQuantFunction``,
``FakeTensorQuantFunction``, ``FakeAffineTensorQuantFunction``) and utils/reduce_amax.py.  Symmetric scaled quantisation maps
``[-amax, amax]`` onto the signed integer grid of ``num_bits`` bits (``narrow_range`` drops the most negative code so the
grid is symmetric); the gradient passes through unchanged where ``|x| <= amax`` and is zero where the value was clipped.
"""
from __future__ import annotations

from typing import Any, Dict, Optional, Sequence, Tuple, Union

import torch

Axis = Union[None, int, Sequence[int]]


def reduce_amax(x: torch.Tensor, axis: Axis = None, keepdims: bool = True) -> torch.Tensor:
    """Maximum of ``|x|`` over every dimension EXCEPT those in ``axis`` (``None``: over all, giving a scalar)."""
    a = x.detach().abs()
    if axis is None:
        return a.max()
    keep = {d % x.dim() for d in ((axis,) if isinstance(axis, int) else axis)}
    dims = [d for d in range(x.dim()) if d not in keep]
    return a.amax(dim=dims, keepdim=keepdims) if dims else a


class QuantDescriptor:
    """How one tensor is quantised.

    ``num_bits``; ``axis``: dimension(s) that keep their own scale (``None`` = one scale per tensor); ``amax``: fixed
    clipping maximum (scalar or list; ``None`` = calibrated, or taken from each input when never calibrated);
    ``learn_amax``: ``amax`` is a trained parameter; ``calib_method``: ``"max"`` or ``"histogram"``; ``unsigned``: codes in
    ``[0, 2^bits - 1]`` for non-negative tensors; ``narrow_range``: symmetric signed grid; ``fake_quant``: return the
    de-quantised float tensor (training) instead of integer codes and a scale."""

    _FIELDS = ("num_bits", "name", "fake_quant", "axis", "amax", "learn_amax", "scale_amax", "calib_method", "unsigned",
               "narrow_range")

    def __init__(self, num_bits: int = 8, name: Optional[str] = None, fake_quant: bool = True, axis: Axis = None, amax=None,
                 learn_amax: bool = False, scale_amax: Optional[float] = None, calib_method: str = "max", unsigned: bool = False,
                 narrow_range: bool = False):
        if not isinstance(num_bits, int) or num_bits < 1:
            raise ValueError(f"num_bits must be a positive integer, not {num_bits!r}")
        if calib_method not in ("max", "histogram"):
            raise ValueError("calib_method is 'max' or 'histogram'")
        if learn_amax and amax is None:
            raise ValueError("learn_amax needs an initial amax")
        if learn_amax and axis is not None and not isinstance(amax, (list, tuple)):
            raise ValueError("a learned per-axis amax needs one initial value per slice")
        if amax is not None and not isinstance(amax, (int, float, list, tuple)):
            raise TypeError("amax is a number or a list of numbers")
        self.num_bits, self.name, self.fake_quant, self.axis, self.amax = num_bits, name, fake_quant, axis, amax
        self.learn_amax, self.scale_amax, self.calib_method = learn_amax, scale_amax, calib_method
        self.unsigned, self.narrow_range = unsigned, narrow_range

    def dict(self) -> Dict[str, Any]:
        """The fields that differ from the defaults (what a config file has to say)."""
        base = QuantDescriptor()
        return {k: getattr(self, k) for k in self._FIELDS if getattr(self, k) != getattr(base, k)}

    def to_yaml(self) -> str:
        import yaml

        return yaml.safe_dump(self.dict())

    @classmethod
    def from_yaml(cls, text: str) -> "QuantDescriptor":
        import yaml

        return cls(**(yaml.safe_load(text) or {}))

    def __eq__(self, other) -> bool:
        return isinstance(other, QuantDescriptor) and all(getattr(self, k) == getattr(other, k) for k in self._FIELDS)

    def __repr__(self) -> str:
        parts = [f"{self.num_bits}bit", "fake" if self.fake_quant else "real", f"axis={self.axis}"]
        parts += [f"{k}={v}" for k, v in self.dict().items() if k not in ("num_bits", "fake_quant", "axis")]
        return "QuantDescriptor(" + " ".join(parts) + ")"


ScaledQuantDescriptor = QuantDescriptor

QUANT_DESC_8BIT_PER_TENSOR = QuantDescriptor(num_bits=8)
QUANT_DESC_UNSIGNED_8BIT_PER_TENSOR = QuantDescriptor(num_bits=8, unsigned=True)
QUANT_DESC_8BIT_LINEAR_WEIGHT_PER_ROW = QuantDescriptor(num_bits=8, axis=0)
QUANT_DESC_8BIT_CONV_WEIGHT_PER_CHANNEL = QuantDescriptor(num_bits=8, axis=0)
QUANT_DESC_8BIT_CONVTRANSPOSE_WEIGHT_PER_CHANNEL = QuantDescriptor(num_bits=8, axis=1)


def _bounds(num_bits: int, unsigned: bool, narrow_range: bool) -> Tuple[float, float]:
    hi = 2.0 ** (num_bits - 1 + int(unsigned)) - 1.0
    if unsigned:
        return 0.0, hi
    return (-hi if narrow_range else -hi - 1.0), hi


def _quantize(x: torch.Tensor, amax: torch.Tensor, num_bits: int, unsigned: bool, narrow_range: bool):
    """Integer codes (as floats) and the scale ``codes = x * scale``.  Slices whose ``amax`` is 0 quantise to 0."""
    if unsigned and bool((x.detach() < 0).any()):
        raise ValueError("unsigned quantisation of a tensor with negative values")
    if bool((amax.detach() < 0).any()):
        raise ValueError("negative amax")
    lo, hi = _bounds(num_bits, unsigned, narrow_range)
    amax_f = amax.to(torch.float32)
    tiny = amax_f <= 2.0 ** -24
    scale = hi / torch.where(tiny, torch.ones_like(amax_f), amax_f)
    scale = torch.where(tiny, torch.zeros_like(scale), scale)
    codes = torch.clamp(torch.round(x.to(torch.float32) * scale), lo, hi)
    return codes, scale


class TensorQuantFunction(torch.autograd.Function):
    """``x -> (integer codes, scale)``; ``x ~ codes / scale``."""

    @staticmethod
    def forward(ctx, x, amax, num_bits=8, unsigned=False, narrow_range=True):
        amax = torch.as_tensor(amax, device=x.device)
        ctx.save_for_backward(x.detach().abs() <= amax.to(x.dtype))
        codes, scale = _quantize(x, amax, num_bits, unsigned, narrow_range)
        ctx.mark_non_differentiable(scale)
        return codes.to(x.dtype), scale

    @staticmethod
    def backward(ctx, g_codes, g_scale):
        (inside,) = ctx.saved_tensors
        return g_codes * inside, None, None, None, None


class FakeTensorQuantFunction(torch.autograd.Function):
    """Quantise and de-quantise in one step: the float tensor the integer kernel would see."""

    @staticmethod
    def forward(ctx, x, amax, num_bits=8, unsigned=False, narrow_range=True):
        amax = torch.as_tensor(amax, device=x.device)
        ctx.save_for_backward(x.detach().abs() <= amax.to(x.dtype))
        codes, scale = _quantize(x, amax, num_bits, unsigned, narrow_range)
        safe = torch.where(scale == 0, torch.ones_like(scale), scale)
        return (codes / safe).to(x.dtype)

    @staticmethod
    def backward(ctx, g):
        (inside,) = ctx.saved_tensors
        return g * inside, None, None, None, None


class FakeAffineTensorQuantFunction(torch.autograd.Function):
    """Asymmetric fake quantisation of ``[min_range, max_range]`` with a zero point (activations after ReLU / GELU)."""

    @staticmethod
    def forward(ctx, x, min_range, max_range, num_bits=8):
        min_range = torch.as_tensor(min_range, device=x.device, dtype=torch.float32)
        max_range = torch.as_tensor(max_range, device=x.device, dtype=torch.float32)
        ctx.save_for_backward((x.detach() >= min_range.to(x.dtype)) & (x.detach() <= max_range.to(x.dtype)))
        step = ((max_range - min_range) / (2.0 ** num_bits - 1.0)).clamp_min(1e-12)
        zero = torch.round(min_range / step)
        lo, hi = -(2.0 ** (num_bits - 1)), 2.0 ** (num_bits - 1) - 1.0
        shift = zero - lo  # code lo represents min_range
        codes = torch.clamp(torch.round(x.to(torch.float32) / step) - shift, lo, hi)
        return ((codes + shift) * step).to(x.dtype)

    @staticmethod
    def backward(ctx, g):
        (inside,) = ctx.saved_tensors
        return g * inside, None, None, None


tensor_quant = TensorQuantFunction.apply
fake_tensor_quant = FakeTensorQuantFunction.apply
fake_affine_tensor_quant = FakeAffineTensorQuantFunction.apply

__all__ = ["QuantDescriptor", "ScaledQuantDescriptor", "reduce_amax", "TensorQuantFunction", "FakeTensorQuantFunction",
           "FakeAffineTensorQuantFunction", "tensor_quant", "fake_tensor_quant", "fake_affine_tensor_quant",
           "QUANT_DESC_8BIT_PER_TENSOR", "QUANT_DESC_UNSIGNED_8BIT_PER_TENSOR", "QUANT_DESC_8BIT_LINEAR_WEIGHT_PER_ROW",
           "QUANT_DESC_8BIT_CONV_WEIGHT_PER_CHANNEL", "QUANT_DESC_8BIT_CONVTRANSPOSE_WEIGHT_PER_CHANNEL"]
