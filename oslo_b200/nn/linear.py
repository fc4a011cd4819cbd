"""Linear layers: plain, GPT-2 ``Conv1D``, and the tensor-parallel variants.

Every layer computes through :func:`oslo_b200.ops.gemm.linear`, i.e. the tcgen05
kernel on CUDA bf16/fp16 and ``F.linear`` elsewhere.  ``skip_bias_add=True``
returns ``(out, bias)`` so the caller can fuse the bias into the next op.

1-D layers accept ``sequence_parallel=True`` (not in the reference): activations
outside the linears are sharded over the flattened token dimension and the layer
performs all-gather->GEMM (column) or GEMM->reduce-scatter (row).

Parity: ``oslo/torch/nn/modules/linear.py:12-535``.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple, Union

import torch
import torch.nn as nn
from torch import Tensor

from oslo_b200.distributed import ParallelMode
from oslo_b200.ops.gemm import linear as _linear


class Linear(nn.Linear):
    #: True when the weight is stored ``[in, out]`` (GPT-2 ``Conv1D`` layout); it is then used through
    #: a transposed view, which the GEMM kernel reads as an MN-major operand without copying.
    reversed = False

    def __init__(self, in_features, out_features, bias=True, dtype=None, skip_bias_add=False, device=None):
        super().__init__(in_features, out_features, bias=bias, device=device, dtype=dtype)
        self.skip_bias_add = skip_bias_add

    @property
    def _w(self):
        return self.weight.t() if self.reversed else self.weight

    def forward(self, input: Tensor) -> Union[Tensor, Tuple[Tensor, Tensor]]:
        if self.skip_bias_add:
            return _linear(input, self._w), self.bias
        return _linear(input, self._w, self.bias)


def _sp_dim(module) -> int:
    st = getattr(module, "sequence_parallel_state", None)
    return st.dim if st is not None else 0


class ColLinear1D(Linear):
    """Weight ``[out/tp, in]``.  Output is sharded on the last dim unless ``gather_output``."""

    def __init__(
        self,
        in_features,
        out_features,
        bias=True,
        dtype=None,
        skip_bias_add=False,
        gather_output=False,
        parallel_context=None,
        sequence_parallel=False,
        device=None,
    ):
        self.gather_output = gather_output
        self.parallel_context = parallel_context
        self.sequence_parallel = sequence_parallel
        self.reversed = False
        self.world_size = parallel_context.get_world_size(ParallelMode.TENSOR_1D)
        if out_features % self.world_size:
            raise ValueError("out_features must be divisible by the tensor-parallel size for ColLinear1D")
        super().__init__(in_features, out_features // self.world_size, bias=bias, dtype=dtype,
                         skip_bias_add=skip_bias_add, device=device)

    def extra_repr(self):
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"gather_output={self.gather_output}, sequence_parallel={self.sequence_parallel}")

    def forward(self, input: Tensor):
        from oslo_b200.parallel.tensor_parallel import _ops_1d as ops

        if self.sequence_parallel and self.world_size > 1:
            # input: token-sharded [..., T/tp, in]; gather over flattened tokens
            lead = list(input.shape[:-1])
            x2 = input.reshape(-1, input.shape[-1])
            fuse_bias = self.bias is not None and not self.skip_bias_add
            out = ops.ag_linear(x2, self._w, self.parallel_context, self.bias if fuse_bias else None)
            if len(lead) > 1:
                d = _sp_dim(self)
                if d != 0 and any(n != 1 for n in lead[:d]):
                    raise ValueError("sequence parallelism over dim 1 needs batch size 1 per rank")
                lead[d] *= self.world_size
                out = out.view(*lead, out.shape[-1])
        else:
            x = ops.broadcast_tensor_1d(input, self.parallel_context)
            if self.bias is not None and not self.skip_bias_add:
                out = _linear(x, self._w, self.bias)
            else:
                out = _linear(x, self._w)
        if self.gather_output:
            out = ops.gather_tensor_1d(out, -1, self.parallel_context)
            if hasattr(self, "orig_num_classes"):
                out = out[..., : self.orig_num_classes]
            out = out.contiguous()
        if self.bias is not None and self.skip_bias_add:
            # the caller adds the bias to what it got: the full width when the output was gathered
            bias = ops.gather_tensor_1d(self.bias, -1, self.parallel_context) if self.gather_output else self.bias
            return out, bias
        return out


class RowLinear1D(Linear):
    """Weight ``[out, in/tp]``.  Input is expected sharded on the last dim (``parallel_input``)."""

    def __init__(
        self,
        in_features,
        out_features,
        bias=True,
        dtype=None,
        skip_bias_add=False,
        parallel_input=True,
        parallel_context=None,
        sequence_parallel=False,
        device=None,
    ):
        self.parallel_input = parallel_input
        self.parallel_context = parallel_context
        self.sequence_parallel = sequence_parallel
        self.reversed = False
        self.world_size = parallel_context.get_world_size(ParallelMode.TENSOR_1D)
        if in_features % self.world_size:
            raise ValueError("in_features must be divisible by the tensor-parallel size for RowLinear1D")
        super().__init__(in_features // self.world_size, out_features, bias=bias, dtype=dtype,
                         skip_bias_add=skip_bias_add, device=device)

    def extra_repr(self):
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"parallel_input={self.parallel_input}, sequence_parallel={self.sequence_parallel}")

    def forward(self, input: Tensor):
        from oslo_b200.parallel.tensor_parallel import _ops_1d as ops

        if not self.parallel_input:
            input = ops.scatter_tensor_1d(input, -1, self.parallel_context)
        if self.sequence_parallel and self.world_size > 1:
            lead = list(input.shape[:-1])
            x2 = input.reshape(-1, input.shape[-1])
            out = ops.linear_rs(x2, self._w, self.parallel_context)
            if len(lead) > 1:
                d = _sp_dim(self)
                if d != 0 and any(n != 1 for n in lead[:d]):
                    raise ValueError("sequence parallelism over dim 1 needs batch size 1 per rank")
                lead[d] //= self.world_size
                out = out.view(*lead, out.shape[-1])
        else:
            out = _linear(input, self._w)
            out = ops.reduce_tensor_1d(out, self.parallel_context)
        if self.bias is not None:
            if self.skip_bias_add:
                return out, self.bias
            return out + self.bias
        return out


# ------------------------------------------------------------------------------ 2D
class Linear2D(Linear):
    """SUMMA linear.  Weight ``[out/q, in/q]``, bias ``[out/q^2]`` (reference linear.py:163-305)."""

    def __init__(self, in_features, out_features, bias=True, dtype=None, skip_bias_add=False,
                 gather_output=False, parallel_context=None, device=None):
        self.parallel_context = parallel_context
        self.gather_output = gather_output
        self.summa_dim = parallel_context.summa_dim
        self.reversed = False
        q = self.summa_dim
        if in_features % q or out_features % (q * q):
            raise ValueError("Linear2D: in_features % q and out_features % q^2 must be 0")
        self.row_rank = parallel_context.get_local_rank(ParallelMode.TENSOR_2D_COL)
        self.col_rank = parallel_context.get_local_rank(ParallelMode.TENSOR_2D_ROW)
        nn.Module.__init__(self)
        self.in_features, self.out_features = in_features // q, out_features // q
        self.skip_bias_add = skip_bias_add
        kw = dict(device=device, dtype=dtype)
        self.weight = nn.Parameter(torch.empty(self.out_features, self.in_features, **kw))
        self.bias = nn.Parameter(torch.empty(out_features // (q * q), **kw)) if bias else None
        self.reset_parameters()

    def reset_parameters(self):
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            bound = 1 / math.sqrt(self.in_features * self.summa_dim)
            nn.init.uniform_(self.bias, -bound, bound)

    def forward(self, input: Tensor):
        from oslo_b200.parallel.tensor_parallel import _ops_2d as ops

        pc = self.parallel_context
        out = ops.matmul_abt_2d(input, self._w, pc)
        if self.bias is not None:
            if self.skip_bias_add:
                return out, ops.gather_bias_2d(self.bias, pc)
            out = ops.add_bias_2d(out, self.bias, pc)
        if self.gather_output:
            out = ops.gather_output_2d(out, pc)
            if hasattr(self, "orig_num_classes"):
                out = out[..., : self.orig_num_classes].contiguous()
        return out


# ---------------------------------------------------------------------------- 2.5D
class Linear2p5D(Linear):
    """Tesseract linear.  Weight ``[out/q, in/q]``, bias ``[out/q]`` (reference linear.py:308-450)."""

    def __init__(self, in_features, out_features, bias=True, dtype=None, skip_bias_add=False,
                 gather_output=False, parallel_context=None, device=None):
        self.parallel_context = parallel_context
        self.gather_output = gather_output
        self.tesseract_dim = parallel_context.summa_dim
        self.tesseract_dep = parallel_context.tensor_parallel_depth
        self.reversed = False
        q = self.tesseract_dim
        if in_features % q or out_features % q:
            raise ValueError("Linear2p5D: in_features % q and out_features % q must be 0")
        nn.Module.__init__(self)
        self.in_features, self.out_features = in_features // q, out_features // q
        self.skip_bias_add = skip_bias_add
        kw = dict(device=device, dtype=dtype)
        self.weight = nn.Parameter(torch.empty(self.out_features, self.in_features, **kw))
        self.bias = nn.Parameter(torch.empty(self.out_features, **kw)) if bias else None
        self.reset_parameters()

    def reset_parameters(self):
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            bound = 1 / math.sqrt(self.in_features * self.tesseract_dim)
            nn.init.uniform_(self.bias, -bound, bound)

    def forward(self, input: Tensor):
        from oslo_b200.parallel.tensor_parallel import _ops_2p5d as ops

        pc = self.parallel_context
        out = ops.matmul_abt_2p5d(input, self._w, pc)
        if self.bias is not None:
            if self.skip_bias_add:
                return out, self.bias
            out = out + self.bias
        if self.gather_output:
            out = ops.gather_output_2p5d(out, pc)
            if hasattr(self, "orig_num_classes"):
                out = out[..., : self.orig_num_classes].contiguous()
        return out


# ------------------------------------------------------------------------------ 3D
class Linear3D(Linear):
    """Cubic linear.  Weight ``[out/c^2, in/c]``, bias ``[out/c]`` (reference linear.py:453-535)."""

    def __init__(self, in_features, out_features, bias=True, dtype=None, skip_bias_add=False,
                 gather_output=False, parallel_context=None, device=None):
        self.parallel_context = parallel_context
        self.gather_output = gather_output
        self.cubic_dim = parallel_context.cubic_dim
        self.reversed = False
        c = self.cubic_dim
        if in_features % c or out_features % (c * c):
            raise ValueError("Linear3D: in_features % c and out_features % c^2 must be 0")
        nn.Module.__init__(self)
        self.in_features, self.out_features = in_features // c, out_features // (c * c)
        self.skip_bias_add = skip_bias_add
        kw = dict(device=device, dtype=dtype)
        self.weight = nn.Parameter(torch.empty(self.out_features, self.in_features, **kw))
        self.bias = nn.Parameter(torch.empty(out_features // c, **kw)) if bias else None
        self.reset_parameters()

    def reset_parameters(self):
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            bound = 1 / math.sqrt(self.in_features * self.cubic_dim)
            nn.init.uniform_(self.bias, -bound, bound)

    def forward(self, input: Tensor):
        from oslo_b200.parallel.tensor_parallel import _ops_3d as ops

        pc = self.parallel_context
        out = ops.linear_3d(input, self._w, None if self.skip_bias_add else self.bias, pc)
        if self.bias is not None and self.skip_bias_add:
            # the output's feature block is this rank's OUTPUT index after the final exchange, while the stored
            # bias block follows the INPUT index: fetch the matching block from the exchange partner
            return out, ops.transpose_3d(self.bias, pc)
        if self.gather_output:
            out = ops.gather_output_3d(out, pc)
            if hasattr(self, "orig_num_classes"):
                out = out[..., : self.orig_num_classes].contiguous()
        return out
