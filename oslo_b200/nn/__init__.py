"""Layer zoo (parity: oslo/torch/nn/__init__.py:1-53)."""
from .conv import Conv1D
from .dropout import FusedBiasDropout
from .embedding import (
    Embedding,
    Embedding1D,
    Embedding2D,
    Embedding2p5D,
    Embedding3D,
    VocabParallelEmbedding1D,
    VocabParallelEmbedding2D,
    VocabParallelEmbedding2p5D,
    VocabParallelEmbedding3D,
    VocabUtility,
)
from .functional import (
    bias_dropout_add,
    bias_gelu,
    fused_bias_dropout,
    fused_bias_gelu,
    fused_gelu,
    fused_layer_norm,
    fused_layer_norm_affine,
    fused_rms_norm,
    fused_rms_norm_affine,
    mixed_dtype_fused_layer_norm_affine,
    mixed_dtype_fused_rms_norm_affine,
    swiglu,
)
from .layer_norm import (
    FusedLayerNorm,
    FusedRMSNorm,
    LayerNorm1D,
    LayerNorm2D,
    LayerNorm2p5D,
    LayerNorm3D,
    MixedFusedLayerNorm,
    MixedFusedRMSNorm,
    RMSNorm1D,
)
from .linear import ColLinear1D, Linear, Linear2D, Linear2p5D, Linear3D, RowLinear1D
from .loss import (
    CrossEntropyLoss2D,
    CrossEntropyLoss2p5D,
    CrossEntropyLoss3D,
    VocabParallelCrossEntropyLoss1D,
    VocabParallelCrossEntropyLoss2D,
    VocabParallelCrossEntropyLoss2p5D,
)
from .zero_linear import ZeroShardedLinear, shard_linears, zero_linear
from .ngram_repeat_block import FusedNoRepeatNGramLogitsProcessor, NGramRepeatBlock, fused_no_repeat_ngram_logits_processor
