"""LayerNorm / RMSNorm modules: fused single-device kernels and the tensor-parallel variants.

* ``FusedLayerNorm`` / ``FusedRMSNorm`` (+ ``MixedFused*`` with fp32 parameters) run
  ``csrc/norm_sm100a.cu`` on CUDA.
* ``LayerNorm1D`` is a replicated LayerNorm that remembers its parallel context; under
  sequence parallelism its parameter gradients are partial sums over token shards and are
  marked (``sequence_parallel_grad``) for the all-reduce done by the TP wrapper.
* ``LayerNorm2D/2p5D/3D`` normalise a hidden dimension that is sharded across ranks:
  the row sums of x and x^2 are all-reduced over the group that holds the hidden shards.

Parity: oslo/torch/nn/modules/layer_norm.py:73-621.
"""
from __future__ import annotations

import numbers

import torch
import torch.nn as nn
from torch.nn import init

from oslo_b200.distributed import ParallelMode
from oslo_b200.ops.norm import layer_norm, rms_norm


def _shape(normalized_shape):
    if isinstance(normalized_shape, numbers.Integral):
        return (int(normalized_shape),)
    return tuple(normalized_shape)


class FusedLayerNorm(nn.Module):
    def __init__(self, normalized_shape, eps=1e-5, elementwise_affine=True, dtype=None, device=None):
        super().__init__()
        self.normalized_shape = _shape(normalized_shape)
        self.eps = eps
        self.elementwise_affine = elementwise_affine
        if elementwise_affine:
            self.weight = nn.Parameter(torch.ones(self.normalized_shape, dtype=dtype, device=device))
            self.bias = nn.Parameter(torch.zeros(self.normalized_shape, dtype=dtype, device=device))
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)

    def forward(self, input):
        return layer_norm(input, self.normalized_shape, self.weight, self.bias, self.eps)

    def extra_repr(self):
        return f"{self.normalized_shape}, eps={self.eps}, elementwise_affine={self.elementwise_affine}"


class FusedRMSNorm(nn.Module):
    def __init__(self, normalized_shape, eps=1e-5, elementwise_affine=True, dtype=None, device=None):
        super().__init__()
        self.normalized_shape = _shape(normalized_shape)
        self.eps = eps
        self.elementwise_affine = elementwise_affine
        if elementwise_affine:
            self.weight = nn.Parameter(torch.ones(self.normalized_shape, dtype=dtype, device=device))
        else:
            self.register_parameter("weight", None)

    def forward(self, input):
        return rms_norm(input, self.normalized_shape, self.weight, self.eps)

    def extra_repr(self):
        return f"{self.normalized_shape}, eps={self.eps}, elementwise_affine={self.elementwise_affine}"


class MixedFusedLayerNorm(FusedLayerNorm):
    """fp32 parameters with fp16 / bf16 activations; output in the activation dtype."""

    def __init__(self, normalized_shape, eps=1e-5, **kwargs):
        kwargs.pop("elementwise_affine", None)
        super().__init__(normalized_shape, eps=eps, elementwise_affine=True, dtype=torch.float32, **kwargs)


class MixedFusedRMSNorm(FusedRMSNorm):
    def __init__(self, normalized_shape, eps=1e-5, **kwargs):
        kwargs.pop("elementwise_affine", None)
        super().__init__(normalized_shape, eps=eps, elementwise_affine=True, dtype=torch.float32, **kwargs)


class LayerNorm1D(FusedLayerNorm):
    def __init__(self, normalized_shape, eps=1e-5, bias=True, dtype=None, parallel_context=None, device=None):
        super().__init__(normalized_shape, eps=eps, elementwise_affine=True, dtype=dtype, device=device)
        if not bias:
            self.bias = None
        self.parallel_context = parallel_context


class RMSNorm1D(FusedRMSNorm):
    def __init__(self, normalized_shape, eps=1e-5, dtype=None, parallel_context=None, device=None):
        super().__init__(normalized_shape, eps=eps, elementwise_affine=True, dtype=dtype, device=device)
        self.parallel_context = parallel_context


class _ShardedNormBase(nn.Module):
    """Normalisation over a hidden dim of global size ``normalized_shape`` sharded over ``self.partitions``."""

    partitions: int
    reduce_mode: ParallelMode

    def _setup(self, normalized_shape, partitioned_dim, eps, bias, dtype, device, rms=False):
        self.normalized_shape = normalized_shape
        self.partitioned_dim = partitioned_dim
        self.variance_epsilon = eps
        self.rms = rms
        kw = dict(dtype=dtype, device=device)
        self.weight = nn.Parameter(torch.ones(partitioned_dim, **kw))
        self.bias = nn.Parameter(torch.zeros(partitioned_dim, **kw)) if (bias and not rms) else None

    def _full_affine(self):
        return self.weight, self.bias

    def forward(self, input):
        from oslo_b200.parallel.tensor_parallel._ops_nd import sharded_norm

        w, b = self._full_affine()
        return sharded_norm(input, w, b, self.normalized_shape, self.variance_epsilon, self.rms,
                            self.parallel_context, self.reduce_mode)

    def extra_repr(self):
        return f"{self.normalized_shape}, partitioned_dim={self.partitioned_dim}, eps={self.variance_epsilon}"


class LayerNorm2D(_ShardedNormBase):
    """Hidden dim split ``q^2`` ways for parameters, ``q`` ways (over the ROW group) for activations."""

    def __init__(self, normalized_shape, eps=1e-5, bias=True, dtype=None, parallel_context=None, device=None):
        super().__init__()
        self.parallel_context = parallel_context
        q = parallel_context.summa_dim
        self.summa_dim = q
        if normalized_shape % (q * q):
            raise ValueError("LayerNorm2D: normalized_shape must be divisible by q^2")
        self.reduce_mode = ParallelMode.TENSOR_2D_ROW
        self._setup(normalized_shape, normalized_shape // (q * q), eps, bias, dtype, device)

    def _full_affine(self):
        from oslo_b200.parallel.tensor_parallel import _ops_2d as ops

        w = ops.gather_bias_2d(self.weight, self.parallel_context)
        b = ops.gather_bias_2d(self.bias, self.parallel_context) if self.bias is not None else None
        return w, b


class LayerNorm2p5D(_ShardedNormBase):
    def __init__(self, normalized_shape, eps=1e-5, bias=True, dtype=None, parallel_context=None, device=None):
        super().__init__()
        self.parallel_context = parallel_context
        q = parallel_context.summa_dim
        self.tesseract_dim = q
        if normalized_shape % q:
            raise ValueError("LayerNorm2p5D: normalized_shape must be divisible by q")
        self.reduce_mode = ParallelMode.TENSOR_2P5D_ROW
        self._setup(normalized_shape, normalized_shape // q, eps, bias, dtype, device)


class LayerNorm3D(_ShardedNormBase):
    def __init__(self, normalized_shape, eps=1e-5, bias=True, dtype=None, parallel_context=None, device=None):
        super().__init__()
        self.parallel_context = parallel_context
        c = parallel_context.cubic_dim
        self.cubic_dim = c
        if normalized_shape % c:
            raise ValueError("LayerNorm3D: normalized_shape must be divisible by c")
        self.reduce_mode = ParallelMode.TENSOR_3D_OUTPUT
        self._setup(normalized_shape, normalized_shape // c, eps, bias, dtype, device)
