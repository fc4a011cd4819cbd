"""Minimal model configuration objects, JSON-compatible with Hugging Face ``config.json`` files.

The attribute names follow the Hugging Face configs of the same families (GPT2Config, GPTNeoXConfig,
LlamaConfig) so a ``config.json`` written here loads there and vice versa; no network or ``transformers``
import is needed.
"""
from __future__ import annotations

import copy
import json
import os
from typing import Any, Dict


class PretrainedConfig:
    model_type = "base"
    architectures = None

    def __init__(self, **kwargs):
        self.torch_dtype = kwargs.pop("torch_dtype", None)
        self.tie_word_embeddings = kwargs.pop("tie_word_embeddings", True)
        self.architectures = kwargs.pop("architectures", None)
        for k, v in kwargs.items():
            setattr(self, k, v)

    def to_dict(self) -> Dict[str, Any]:
        out = {}
        for k, v in copy.deepcopy(self.__dict__).items():
            if k.startswith("_"):
                continue
            if k == "torch_dtype" and v is not None:
                v = str(v).replace("torch.", "")
            out[k] = v
        out["model_type"] = self.model_type
        return out

    def to_json_string(self) -> str:
        return json.dumps(self.to_dict(), indent=2, sort_keys=True) + "\n"

    def save_pretrained(self, save_directory: str):
        os.makedirs(save_directory, exist_ok=True)
        with open(os.path.join(save_directory, "config.json"), "w") as f:
            f.write(self.to_json_string())

    @classmethod
    def from_dict(cls, d: Dict[str, Any]):
        d = dict(d)
        d.pop("model_type", None)
        return cls(**d)

    @classmethod
    def from_pretrained(cls, path: str):
        file = os.path.join(path, "config.json") if os.path.isdir(path) else path
        with open(file) as f:
            return cls.from_dict(json.load(f))

    def __repr__(self):
        return f"{self.__class__.__name__} {self.to_json_string()}"


class GPT2Config(PretrainedConfig):
    model_type = "gpt2"

    def __init__(self, vocab_size=50257, n_positions=1024, n_embd=768, n_layer=12, n_head=12, n_inner=None,
                 activation_function="gelu_new", resid_pdrop=0.1, embd_pdrop=0.1, attn_pdrop=0.1,
                 layer_norm_epsilon=1e-5, initializer_range=0.02, **kwargs):
        self.vocab_size, self.n_positions, self.n_embd = vocab_size, n_positions, n_embd
        self.n_layer, self.n_head, self.n_inner = n_layer, n_head, n_inner
        self.activation_function = activation_function
        self.resid_pdrop, self.embd_pdrop, self.attn_pdrop = resid_pdrop, embd_pdrop, attn_pdrop
        self.layer_norm_epsilon, self.initializer_range = layer_norm_epsilon, initializer_range
        super().__init__(**kwargs)

    hidden_size = property(lambda self: self.n_embd)
    num_hidden_layers = property(lambda self: self.n_layer)
    num_attention_heads = property(lambda self: self.n_head)


class GPTNeoXConfig(PretrainedConfig):
    model_type = "gpt_neox"

    def __init__(self, vocab_size=50432, hidden_size=6144, num_hidden_layers=44, num_attention_heads=64,
                 intermediate_size=24576, hidden_act="gelu", rotary_pct=0.25, rotary_emb_base=10000,
                 max_position_embeddings=2048, initializer_range=0.02, layer_norm_eps=1e-5,
                 use_parallel_residual=True, hidden_dropout=0.0, attention_dropout=0.0, **kwargs):
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.num_hidden_layers, self.num_attention_heads = num_hidden_layers, num_attention_heads
        self.intermediate_size, self.hidden_act = intermediate_size, hidden_act
        self.rotary_pct, self.rotary_emb_base = rotary_pct, rotary_emb_base
        self.max_position_embeddings = max_position_embeddings
        self.initializer_range, self.layer_norm_eps = initializer_range, layer_norm_eps
        self.use_parallel_residual = use_parallel_residual
        self.hidden_dropout, self.attention_dropout = hidden_dropout, attention_dropout
        kwargs.setdefault("tie_word_embeddings", False)
        super().__init__(**kwargs)


class LlamaConfig(PretrainedConfig):
    model_type = "llama"

    def __init__(self, vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
                 num_attention_heads=32, num_key_value_heads=None, hidden_act="silu", max_position_embeddings=2048,
                 initializer_range=0.02, rms_norm_eps=1e-6, rope_theta=10000.0, **kwargs):
        self.vocab_size, self.hidden_size, self.intermediate_size = vocab_size, hidden_size, intermediate_size
        self.num_hidden_layers, self.num_attention_heads = num_hidden_layers, num_attention_heads
        self.num_key_value_heads = num_key_value_heads or num_attention_heads
        self.hidden_act, self.max_position_embeddings = hidden_act, max_position_embeddings
        self.initializer_range, self.rms_norm_eps, self.rope_theta = initializer_range, rms_norm_eps, rope_theta
        kwargs.setdefault("tie_word_embeddings", False)
        super().__init__(**kwargs)


class MoEGPTConfig(GPT2Config):
    """GPT-2 style decoder where every ``moe_every`` -th FFN is a mixture of experts."""

    model_type = "moe_gpt"

    def __init__(self, num_experts=16, moe_every=2, top_k=2, capacity_factor=1.25, aux_loss_coef=0.01, **kwargs):
        self.num_experts, self.moe_every, self.top_k = num_experts, moe_every, top_k
        self.capacity_factor, self.aux_loss_coef = capacity_factor, aux_loss_coef
        super().__init__(**kwargs)


def _defaults(self, given: Dict[str, Any], **defaults):
    """Set every default as an attribute, overridden by what the caller gave; the rest of ``given`` is returned."""
    for k, v in defaults.items():
        setattr(self, k, given.pop(k, v))
    return given


class BertConfig(PretrainedConfig):
    model_type = "bert"

    def __init__(self, **kwargs):
        kwargs = _defaults(self, kwargs, vocab_size=30522, hidden_size=768, num_hidden_layers=12, num_attention_heads=12,
                           intermediate_size=3072, hidden_act="gelu", hidden_dropout_prob=0.1,
                           attention_probs_dropout_prob=0.1, max_position_embeddings=512, type_vocab_size=2,
                           initializer_range=0.02, layer_norm_eps=1e-12, pad_token_id=0, num_labels=2,
                           classifier_dropout=None)
        super().__init__(**kwargs)


class RobertaConfig(BertConfig):
    model_type = "roberta"

    def __init__(self, **kwargs):
        kwargs.setdefault("vocab_size", 50265)
        kwargs.setdefault("max_position_embeddings", 514)
        kwargs.setdefault("type_vocab_size", 1)
        kwargs.setdefault("pad_token_id", 1)
        super().__init__(**kwargs)


class ElectraConfig(BertConfig):
    model_type = "electra"

    def __init__(self, **kwargs):
        kwargs = _defaults(self, kwargs, embedding_size=128)
        kwargs.setdefault("hidden_size", 256)
        kwargs.setdefault("num_attention_heads", 4)
        kwargs.setdefault("intermediate_size", 1024)
        super().__init__(**kwargs)


class AlbertConfig(PretrainedConfig):
    model_type = "albert"

    def __init__(self, **kwargs):
        kwargs = _defaults(self, kwargs, vocab_size=30000, embedding_size=128, hidden_size=4096, num_hidden_layers=12,
                           num_hidden_groups=1, num_attention_heads=64, intermediate_size=16384, inner_group_num=1,
                           hidden_act="gelu_new", hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0,
                           max_position_embeddings=512, type_vocab_size=2, initializer_range=0.02, layer_norm_eps=1e-12,
                           classifier_dropout_prob=0.1, pad_token_id=0, num_labels=2)
        super().__init__(**kwargs)


class DistilBertConfig(PretrainedConfig):
    model_type = "distilbert"

    def __init__(self, **kwargs):
        kwargs = _defaults(self, kwargs, vocab_size=30522, max_position_embeddings=512, n_layers=6, n_heads=12, dim=768,
                           hidden_dim=3072, dropout=0.1, attention_dropout=0.1, activation="gelu", initializer_range=0.02,
                           qa_dropout=0.1, seq_classif_dropout=0.2, pad_token_id=0, num_labels=2)
        super().__init__(**kwargs)

    hidden_size = property(lambda self: self.dim)
    num_hidden_layers = property(lambda self: self.n_layers)
    num_attention_heads = property(lambda self: self.n_heads)


class BartConfig(PretrainedConfig):
    model_type = "bart"

    def __init__(self, **kwargs):
        kwargs = _defaults(self, kwargs, vocab_size=50265, max_position_embeddings=1024, encoder_layers=12,
                           encoder_ffn_dim=4096, encoder_attention_heads=16, decoder_layers=12, decoder_ffn_dim=4096,
                           decoder_attention_heads=16, activation_function="gelu", d_model=1024, dropout=0.1,
                           attention_dropout=0.0, activation_dropout=0.0, init_std=0.02, classifier_dropout=0.0,
                           scale_embedding=False, pad_token_id=1, bos_token_id=0, eos_token_id=2,
                           decoder_start_token_id=2, num_labels=3)
        super().__init__(**kwargs)
        self.initializer_range = self.init_std

    hidden_size = property(lambda self: self.d_model)
    num_hidden_layers = property(lambda self: self.encoder_layers)
    num_attention_heads = property(lambda self: self.encoder_attention_heads)


class MBartConfig(BartConfig):
    model_type = "mbart"

    def __init__(self, **kwargs):
        kwargs.setdefault("vocab_size", 50265)
        super().__init__(**kwargs)


class T5Config(PretrainedConfig):
    model_type = "t5"

    def __init__(self, **kwargs):
        kwargs = _defaults(self, kwargs, vocab_size=32128, d_model=512, d_kv=64, d_ff=2048, num_layers=6,
                           num_decoder_layers=None, num_heads=8, relative_attention_num_buckets=32,
                           relative_attention_max_distance=128, dropout_rate=0.1, layer_norm_epsilon=1e-6,
                           initializer_factor=1.0, feed_forward_proj="relu", pad_token_id=0, eos_token_id=1,
                           decoder_start_token_id=0)
        if self.num_decoder_layers is None:
            self.num_decoder_layers = self.num_layers
        super().__init__(**kwargs)

    hidden_size = property(lambda self: self.d_model)
    num_hidden_layers = property(lambda self: self.num_layers)
    num_attention_heads = property(lambda self: self.num_heads)
    is_gated_act = property(lambda self: self.feed_forward_proj.startswith("gated-"))
    # "gated-gelu" means the tanh form of GELU (as in the released mT5 / T5 v1.1 checkpoints)
    dense_act_fn = property(lambda self: "gelu_new" if self.feed_forward_proj == "gated-gelu" else self.feed_forward_proj.split("-")[-1])


class MT5Config(T5Config):
    model_type = "mt5"

    def __init__(self, **kwargs):
        kwargs.setdefault("vocab_size", 250112)
        kwargs.setdefault("feed_forward_proj", "gated-gelu")
        kwargs.setdefault("tie_word_embeddings", False)
        super().__init__(**kwargs)
