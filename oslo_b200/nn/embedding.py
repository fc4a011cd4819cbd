"""Embeddings: plain, hidden-sharded and vocab-parallel for every tensor-parallel mode.

Parity: oslo/torch/nn/modules/embedding.py:11-506.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from oslo_b200.distributed import ParallelMode


class VocabUtility:
    """Vocabulary range ``[first, last)`` owned by a rank."""

    @staticmethod
    def vocab_range_from_per_partition_vocab_size(per_partition_vocab_size, rank, world_size=None):
        first = rank * per_partition_vocab_size
        return first, first + per_partition_vocab_size

    @staticmethod
    def vocab_range_from_global_vocab_size(global_vocab_size, rank, world_size):
        assert global_vocab_size % world_size == 0
        return VocabUtility.vocab_range_from_per_partition_vocab_size(global_vocab_size // world_size, rank)


class Embedding(nn.Embedding):
    pass


def _masked_lookup(ids, weight, start, end, padding_idx=None):
    mask = (ids < start) | (ids >= end)
    local = (ids - start).masked_fill(mask, 0)
    out = F.embedding(local, weight)
    return out.masked_fill(mask.unsqueeze(-1), 0)


class Embedding1D(nn.Embedding):
    """Hidden dim split over TP; output gathered on the last dim unless ``gather_output`` is off (a per-head table such as
    T5's relative attention bias, whose consumer works on the local heads)."""

    gather_output = True

    def __init__(self, num_embeddings, embedding_dim, dtype=None, parallel_context=None, device=None, gather_output=True, **kw):
        self.parallel_context = parallel_context
        self.gather_output = gather_output
        self.world_size = parallel_context.get_world_size(ParallelMode.TENSOR_1D)
        assert embedding_dim % self.world_size == 0
        super().__init__(num_embeddings, embedding_dim // self.world_size, dtype=dtype, device=device, **kw)

    def forward(self, input):
        from oslo_b200.parallel.tensor_parallel import _ops_1d as ops

        out = F.embedding(input, self.weight, self.padding_idx)
        return ops.gather_tensor_1d(out, -1, self.parallel_context) if self.gather_output else out


class VocabParallelEmbedding1D(nn.Embedding):
    """Vocabulary rows split over TP: masked local lookup then all-reduce (or reduce-scatter under SP)."""

    def __init__(self, num_embeddings, embedding_dim, dtype=None, parallel_context=None, sequence_parallel=False,
                 device=None, **kw):
        self.parallel_context = parallel_context
        self.sequence_parallel = sequence_parallel
        rank = parallel_context.get_local_rank(ParallelMode.TENSOR_1D)
        self.world_size = parallel_context.get_world_size(ParallelMode.TENSOR_1D)
        assert num_embeddings % self.world_size == 0
        self.vocab_start_index, self.vocab_end_index = VocabUtility.vocab_range_from_global_vocab_size(
            num_embeddings, rank, self.world_size)
        super().__init__(num_embeddings // self.world_size, embedding_dim, dtype=dtype, device=device, **kw)

    def forward(self, input):
        from oslo_b200.parallel.tensor_parallel import _ops_1d as ops

        if self.world_size == 1:
            return F.embedding(input, self.weight)
        sbuf = getattr(self.weight, "oslo_symm", None)
        if sbuf is not None and self.sequence_parallel and input.is_cuda:
            # the table is readable by every rank: look up this rank's token shard straight from the owners
            from oslo_b200.distributed import comm
            from oslo_b200.ops.embedding import embedding_pull

            st = getattr(self, "sequence_parallel_state", None)
            d = st.dim if st is not None else 0
            ids = comm.scatter(input, dim=d, parallel_context=self.parallel_context, parallel_mode=ParallelMode.TENSOR_1D)
            return embedding_pull(ids, self.weight, sbuf, self.parallel_context, ParallelMode.TENSOR_1D)
        out = _masked_lookup(input, self.weight, self.vocab_start_index, self.vocab_end_index)
        if self.sequence_parallel:
            st = getattr(self, "sequence_parallel_state", None)
            d = st.dim if st is not None else 0
            return ops.reduce_scatter_tensor_1d(out, d, self.parallel_context)
        return ops.reduce_tensor_1d(out, self.parallel_context)


# ------------------------------------------------------------------------------ 2D
class Embedding2D(nn.Embedding):
    """Weight ``[V, h/q^2]``; gathered over COL to ``[V, h/q]`` before the lookup."""

    def __init__(self, num_embeddings, embedding_dim, dtype=None, parallel_context=None, device=None, **kw):
        self.parallel_context = parallel_context
        q = parallel_context.summa_dim
        self.summa_dim = q
        assert embedding_dim % (q * q) == 0
        super().__init__(num_embeddings, embedding_dim // (q * q), dtype=dtype, device=device, **kw)

    def forward(self, input):
        from oslo_b200.parallel.tensor_parallel import _ops_2d as ops

        w = ops.all_gather_tensor_2d(self.weight, -1, ParallelMode.TENSOR_2D_COL, self.parallel_context)
        return F.embedding(input, w, self.padding_idx)


class VocabParallelEmbedding2D(nn.Embedding):
    """Weight ``[V/q, h/q]``: ids gathered over COL, masked lookup, reduce-scatter over COL on the batch dim."""

    def __init__(self, num_embeddings, embedding_dim, dtype=None, parallel_context=None, device=None, **kw):
        self.parallel_context = parallel_context
        q = parallel_context.summa_dim
        self.summa_dim = q
        assert num_embeddings % q == 0 and embedding_dim % q == 0
        rank = parallel_context.get_local_rank(ParallelMode.TENSOR_2D_COL)
        self.vocab_start_index = rank * (num_embeddings // q)
        self.vocab_end_index = self.vocab_start_index + num_embeddings // q
        super().__init__(num_embeddings // q, embedding_dim // q, dtype=dtype, device=device, **kw)

    def forward(self, input):
        from oslo_b200.parallel.tensor_parallel import _ops_2d as ops

        pc = self.parallel_context
        ids = ops.gather_batch_2d(input, pc)
        out = _masked_lookup(ids, self.weight, self.vocab_start_index, self.vocab_end_index)
        return ops.reduce_scatter_tensor_2d(out, 0, ParallelMode.TENSOR_2D_COL, pc)


# ---------------------------------------------------------------------------- 2.5D
class Embedding2p5D(nn.Embedding):
    def __init__(self, num_embeddings, embedding_dim, dtype=None, parallel_context=None, device=None, **kw):
        self.parallel_context = parallel_context
        q = parallel_context.summa_dim
        self.tesseract_dim = q
        assert embedding_dim % (q * q) == 0
        super().__init__(num_embeddings, embedding_dim // (q * q), dtype=dtype, device=device, **kw)

    def forward(self, input):
        from oslo_b200.parallel.tensor_parallel import _ops_2p5d as ops

        w = ops.all_gather_tensor_2p5d(self.weight, -1, ParallelMode.TENSOR_2P5D_COL, self.parallel_context)
        return F.embedding(input, w, self.padding_idx)


class VocabParallelEmbedding2p5D(nn.Embedding):
    def __init__(self, num_embeddings, embedding_dim, dtype=None, parallel_context=None, device=None, **kw):
        self.parallel_context = parallel_context
        q = parallel_context.summa_dim
        self.tesseract_dim = q
        assert num_embeddings % q == 0 and embedding_dim % q == 0
        rank = parallel_context.get_local_rank(ParallelMode.TENSOR_2P5D_COL)
        self.vocab_start_index = rank * (num_embeddings // q)
        self.vocab_end_index = self.vocab_start_index + num_embeddings // q
        super().__init__(num_embeddings // q, embedding_dim // q, dtype=dtype, device=device, **kw)

    def forward(self, input):
        from oslo_b200.parallel.tensor_parallel import _ops_2p5d as ops

        pc = self.parallel_context
        ids = ops.gather_batch_2p5d(input, pc)
        out = _masked_lookup(ids, self.weight, self.vocab_start_index, self.vocab_end_index)
        return ops.reduce_scatter_tensor_2p5d(out, 0, ParallelMode.TENSOR_2P5D_COL, pc)


# ------------------------------------------------------------------------------ 3D
class Embedding3D(nn.Embedding):
    """Weight ``[V, h/c]`` replicated along INPUT/WEIGHT (kept equal by broadcasting the gradient sum)."""

    def __init__(self, num_embeddings, embedding_dim, dtype=None, parallel_context=None, device=None, **kw):
        self.parallel_context = parallel_context
        c = parallel_context.cubic_dim
        self.cubic_dim = c
        assert embedding_dim % c == 0
        super().__init__(num_embeddings, embedding_dim // c, dtype=dtype, device=device, **kw)

    def forward(self, input):
        from oslo_b200.parallel.tensor_parallel import _ops_3d as ops

        w = ops.replicated_weight_3d(self.weight, self.parallel_context)
        return F.embedding(input, w, self.padding_idx)


class VocabParallelEmbedding3D(nn.Embedding):
    """Weight ``[V/c^2, h/c]``: vocab split over (INPUT, WEIGHT), hidden over OUTPUT."""

    def __init__(self, num_embeddings, embedding_dim, dtype=None, parallel_context=None, device=None, **kw):
        self.parallel_context = parallel_context
        c = parallel_context.cubic_dim
        self.cubic_dim = c
        assert num_embeddings % (c * c) == 0 and embedding_dim % c == 0
        in_rank = parallel_context.get_local_rank(ParallelMode.TENSOR_3D_INPUT)
        self.vocab_per_input = num_embeddings // c
        self.vocab_start_index = in_rank * self.vocab_per_input
        self.vocab_end_index = self.vocab_start_index + self.vocab_per_input
        super().__init__(num_embeddings // (c * c), embedding_dim // c, dtype=dtype, device=device, **kw)

    def forward(self, input):
        from oslo_b200.parallel.tensor_parallel import _ops_3d as ops

        pc = self.parallel_context
        ids = ops.gather_batch_3d(input, ParallelMode.TENSOR_3D_INPUT, pc)
        w = ops.all_gather_weight_3d(self.weight, 0, ParallelMode.TENSOR_3D_WEIGHT, pc)
        out = _masked_lookup(ids, w, self.vocab_start_index, self.vocab_end_index)
        return ops.reduce_scatter_tensor_3d(out, 0, ParallelMode.TENSOR_3D_INPUT, pc)
