from .albert import *  # noqa: F401,F403
from .bart import *  # noqa: F401,F403
from .bert import *  # noqa: F401,F403
from .config import (AlbertConfig, BartConfig, BertConfig, DistilBertConfig, ElectraConfig, GPT2Config, GPTNeoXConfig,
                     LlamaConfig, MBartConfig, MoEGPTConfig, MT5Config, PretrainedConfig, RobertaConfig, T5Config)
from .distilbert import *  # noqa: F401,F403
from .gpt2 import GPT2LMHeadModel, GPT2Model, MoEGPTLMHeadModel
from .gpt_neox import GPTNeoXForCausalLM, GPTNeoXModel
from .llama import LlamaForCausalLM, LlamaModel
from .modeling_utils import CausalLMOutput, ModelOutput, OsloModel, PreTrainedModel
from .t5 import *  # noqa: F401,F403
from . import albert as _albert, bart as _bart, bert as _bert, distilbert as _distilbert, t5 as _t5

__all__ = ["PretrainedConfig", "GPT2Config", "GPTNeoXConfig", "LlamaConfig", "MoEGPTConfig", "BertConfig", "RobertaConfig",
           "ElectraConfig", "AlbertConfig", "DistilBertConfig", "BartConfig", "MBartConfig", "T5Config", "MT5Config",
           "GPT2Model", "GPT2LMHeadModel", "MoEGPTLMHeadModel", "GPTNeoXModel", "GPTNeoXForCausalLM", "LlamaModel",
           "LlamaForCausalLM", "PreTrainedModel", "OsloModel", "CausalLMOutput", "ModelOutput"]
for _m in (_albert, _bart, _bert, _distilbert, _t5):
    __all__ += list(_m.__all__)
