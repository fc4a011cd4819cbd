from .config import GPT2Config, GPTNeoXConfig, LlamaConfig, MoEGPTConfig, PretrainedConfig
from .gpt2 import GPT2LMHeadModel, GPT2Model, MoEGPTLMHeadModel
from .gpt_neox import GPTNeoXForCausalLM, GPTNeoXModel
from .llama import LlamaForCausalLM, LlamaModel
from .modeling_utils import CausalLMOutput, OsloModel, PreTrainedModel

__all__ = ["PretrainedConfig", "GPT2Config", "GPTNeoXConfig", "LlamaConfig", "MoEGPTConfig", "GPT2Model",
           "GPT2LMHeadModel", "MoEGPTLMHeadModel", "GPTNeoXModel", "GPTNeoXForCausalLM", "LlamaModel",
           "LlamaForCausalLM", "PreTrainedModel", "OsloModel", "CausalLMOutput"]
