"""Counterparts of the vendored LightSeq subset of the reference (``oslo/lightseq2``), on this repository's kernels."""
from .gcq import GCQState, gcq_hook, quantized_all_reduce
from .inference import generate
from .kernels import filter_logits, ls_dequantize_int8, ls_embedding, ls_quantize_int8, sample_tokens
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
from .crf import LSCRFLayer
from .export import export_model, import_into, load_exported
from .lsflow_models import LSFlowBert, LSFlowBertCrf, LSFlowGpt, LSFlowTransformer, LSFlowVit
from .models import LSBert, LSBertCrf, LSGpt, LSVit, LSModelConfig, LSTransformer, LSTransformerDecoder, LSTransformerEncoder, get_config
