"""Base class of the in-tree models and the causal-LM output container."""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn


class OsloModel:
    """Marker: models whose heads keep their outputs sharded (the loss is vocab-parallel)."""


@dataclass
class CausalLMOutput:
    loss: Optional[torch.Tensor] = None
    logits: Optional[torch.Tensor] = None
    aux_loss: Optional[torch.Tensor] = None

    def __getitem__(self, k):
        if isinstance(k, str):
            return getattr(self, k)
        return tuple(v for v in (self.loss, self.logits) if v is not None)[k]


class ModelOutput(dict):
    """Named outputs with attribute, key and index access (index skips entries that are ``None``)."""

    def __init__(self, **kw):
        super().__init__(**kw)

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError:
            raise AttributeError(k)

    def __setattr__(self, k, v):
        self[k] = v

    def __getitem__(self, k):
        if isinstance(k, str):
            return dict.__getitem__(self, k)
        return tuple(v for v in self.values() if v is not None)[k]

    def to_tuple(self):
        return tuple(v for v in self.values() if v is not None)


def additive_mask(attention_mask, dtype=torch.float32, tgt_len=None):
    """``[b, s]`` mask of ones (keep) and zeros (padding) -> additive ``[b, 1, tgt or 1, s]`` mask; ``None`` stays."""
    if attention_mask is None:
        return None
    if attention_mask.dim() == 4:
        return attention_mask
    m = (1.0 - attention_mask[:, None, None, :].to(dtype)) * torch.finfo(dtype).min
    return m if tgt_len is None else m.expand(-1, 1, tgt_len, -1)


class PreTrainedModel(nn.Module, OsloModel):
    config_class = None
    base_model_prefix = ""

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.parallel_context = None

    def get_input_embeddings(self):
        raise NotImplementedError

    def get_output_embeddings(self):
        return None

    def tie_weights(self):
        out, inp = self.get_output_embeddings(), self.get_input_embeddings()
        if out is not None and getattr(self.config, "tie_word_embeddings", False):
            out.weight = inp.weight

    def _init_weights(self, module):
        std = getattr(self.config, "initializer_range", 0.02)
        if isinstance(module, nn.Linear) or module.__class__.__name__ == "Conv1D":
            module.weight.data.normal_(mean=0.0, std=std)
            if getattr(module, "bias", None) is not None:
                module.bias.data.zero_()
        elif isinstance(module, nn.Embedding):
            module.weight.data.normal_(mean=0.0, std=std)
        elif isinstance(module, nn.LayerNorm) or module.__class__.__name__ in ("FusedLayerNorm", "FusedRMSNorm"):
            if getattr(module, "bias", None) is not None:
                module.bias.data.zero_()
            module.weight.data.fill_(1.0)

    def post_init(self):
        self.apply(self._init_weights)
        self.tie_weights()

    def num_parameters(self):
        return sum(p.numel() for p in self.parameters())

    def save_pretrained(self, save_directory, save_config=True, state_dict=None, save_function=torch.save, **kw):
        os.makedirs(save_directory, exist_ok=True)
        if save_config:
            self.config.architectures = [self.__class__.__name__]
            self.config.save_pretrained(save_directory)
        save_function(state_dict if state_dict is not None else self.state_dict(),
                      os.path.join(save_directory, "pytorch_model.bin"))

    @classmethod
    def from_pretrained(cls, path, config=None, **kw):
        config = config or cls.config_class.from_pretrained(path)
        model = cls(config)
        state = torch.load(os.path.join(path, "pytorch_model.bin"), map_location="cpu")
        model.load_state_dict(state, strict=False)
        model.tie_weights()
        return model
