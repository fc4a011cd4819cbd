"""Counterparts of the vendored LightSeq subset of the reference (``oslo/lightseq2``), on this repository's kernels."""
from .gcq import GCQState, gcq_hook, quantized_all_reduce
from .inference import generate
from .layers import (
    LSAdam,
    LSCrossEntropyLayer,
    LSGptEncoderLayer,
    LSLayerConfig,
    LSMultiheadAttentionLayer,
    LSTransformerDecoderLayer,
    LSTransformerEmbeddingLayer,
    LSTransformerEncoderLayer,
)
from .memory_planner import ActivationPlan, plan
from .quantization import QuantLinear, TensorQuantizer, quantize_int8
