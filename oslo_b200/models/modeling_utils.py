"""Base class of the in-tree models and the causal-LM output container."""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

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


class Seq2SeqCache:
    """Decoder state of an encoder-decoder model during incremental generation: per attention module the keys / values
    of the target tokens seen so far (self-attention, grown by one position per step) and the projected encoder memory
    (cross-attention, computed on the first step only).  ``offset`` is the number of target tokens already stored; the
    decoders add it to their positions / relative-position biases.  The reference keeps the same buffers in its decoder
    (oslo/lightseq2/inference/model/decoder.cc.cu: self key / value caches per layer, encoder key / value projected once)."""

    def __init__(self):
        self.self_kv: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self.cross_kv: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self.offset = 0

    def self_append(self, key: int, k: torch.Tensor, v: torch.Tensor):
        """``k`` / ``v``: ``[batch, new tokens, heads, head_dim]``; returns everything stored for ``key`` so far."""
        if key in self.self_kv:
            pk, pv = self.self_kv[key]
            k, v = torch.cat([pk, k], dim=1), torch.cat([pv, v], dim=1)
        self.self_kv[key] = (k, v)
        return k, v

    def cross(self, key: int, make):
        if key not in self.cross_kv:
            self.cross_kv[key] = make()
        return self.cross_kv[key]

    def advance(self, n: int):
        self.offset += n

    def reorder(self, index: torch.Tensor):
        """Beam search: hypothesis ``i`` continues hypothesis ``index[i]``."""
        self.self_kv = {k: (a.index_select(0, index), b.index_select(0, index)) for k, (a, b) in self.self_kv.items()}
        self.cross_kv = {k: (a.index_select(0, index), b.index_select(0, index)) for k, (a, b) in self.cross_kv.items()}


_S2S_CACHE: Optional[Seq2SeqCache] = None


class seq2seq_cache:
    """Context manager that makes ``cache`` the active :class:`Seq2SeqCache` (inference only)."""

    def __init__(self, cache: Seq2SeqCache):
        self.cache = cache

    def __enter__(self):
        global _S2S_CACHE
        self.prev, _S2S_CACHE = _S2S_CACHE, self.cache
        return self.cache

    def __exit__(self, *exc):
        global _S2S_CACHE
        _S2S_CACHE = self.prev


def active_seq2seq_cache() -> Optional[Seq2SeqCache]:
    return _S2S_CACHE


def offset_causal_mask(new: int, past: int, device, dtype=torch.float32) -> Optional[torch.Tensor]:
    """Additive ``[new, past + new]`` mask: new token ``i`` sees stored positions ``<= past + i``.  ``None`` when a single
    token is fed (it sees everything)."""
    if new == 1:
        return None
    return torch.full((new, past + new), torch.finfo(dtype).min, device=device, dtype=dtype).triu(past + 1)


@torch.no_grad()
def seq2seq_generate(model, encode, decode_logits, input_ids, attention_mask, max_new_tokens: int, num_beams: int,
                     length_penalty: float, start_id: int, eos_id: int, pad_id: int, use_cache: bool = True):
    """Greedy / beam-search decoding shared by the encoder-decoder models.  ``encode(ids, mask)`` returns the encoder
    output; ``decode_logits(enc, mask, decoder_ids)`` the logits of the LAST fed position.  With ``use_cache`` each step
    feeds only the newest token and the attention modules read their :class:`Seq2SeqCache`."""
    b = input_ids.shape[0]
    dev = input_ids.device
    enc = encode(input_ids, attention_mask)
    if num_beams > 1:
        enc = enc.repeat_interleave(num_beams, dim=0)
        attention_mask = attention_mask.repeat_interleave(num_beams, dim=0) if attention_mask is not None else None
    n = b * num_beams
    out = torch.full((n, 1), start_id, dtype=torch.long, device=dev)
    done = torch.zeros(n, dtype=torch.bool, device=dev)
    scores = torch.zeros(b, num_beams, device=dev)
    if num_beams > 1:
        scores[:, 1:] = -1e9  # the beams start identical: only the first may spawn children at step 0
    cache = Seq2SeqCache() if use_cache else None
    for _ in range(max_new_tokens):
        if cache is not None:
            feed = out[:, cache.offset:]
            with seq2seq_cache(cache):
                logits = decode_logits(enc, attention_mask, feed)
            cache.advance(feed.shape[1])
        else:
            logits = decode_logits(enc, attention_mask, out)
        if getattr(model, "parallel_context", None) is not None:
            from oslo_b200.lightseq.inference import _whole_logits

            logits = _whole_logits(model, logits)  # tensor-parallel heads return a vocabulary shard
        if num_beams == 1:
            nxt = logits.argmax(-1).masked_fill(done, pad_id)
        else:
            logp = torch.log_softmax(logits.float(), dim=-1)
            logp[done] = -1e9
            logp[done, pad_id] = 0.0  # finished hypotheses extend with padding at no cost
            v = logp.shape[-1]
            scores, idx = (scores.view(-1, 1) + logp).view(b, num_beams * v).topk(num_beams, dim=-1)
            parent = (idx // v + torch.arange(b, device=dev).unsqueeze(1) * num_beams).view(-1)
            nxt = (idx % v).view(-1)
            out, done = out[parent], done[parent]
            if cache is not None:
                cache.reorder(parent)
        out = torch.cat([out, nxt[:, None]], dim=1)
        done = done | (nxt == eos_id)
        if bool(done.all()):
            break
    if num_beams > 1:
        lengths = (out != pad_id).sum(-1).view(b, num_beams).float()
        best = (scores / lengths.pow(length_penalty)).argmax(-1)
        out = out.view(b, num_beams, -1)[torch.arange(b, device=dev), best]
    return out
