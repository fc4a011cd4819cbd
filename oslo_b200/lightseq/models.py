"""Whole models assembled from the LightSeq-interface layers: a translation Transformer (encoder + decoder with tied
embeddings and output projection), a decoder-only GPT and a BERT-style encoder with a classification head.

They follow the model classes of the reference's LightSeq subset (training side:
oslo/lightseq2/training/ops/pytorch/transformer.py:15-210; the lsflow models ``Transformer``, ``Gpt``, ``Bert`` of
oslo/lightseq2/csrc/models): configured through ``get_config(model="transformer-base", ...)`` presets, ``forward``
for training and ``infer`` for generation (greedy or beam search; the encoder runs once, the decoder incrementally with
the key / value cache of :mod:`oslo_b200.lightseq.inference`).
"""
from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Optional

import torch
import torch.nn as nn

import oslo_b200.nn as onn

from .layers import (LSCrossEntropyLayer, LSGptEncoderLayer, LSLayerConfig, LSTransformerDecoderLayer,
                     LSTransformerEmbeddingLayer, LSTransformerEncoderLayer)


@dataclass
class LSModelConfig(LSLayerConfig):
    num_encoder_layer: int = 6
    num_decoder_layer: int = 6
    num_labels: int = 2
    bos_id: int = 2
    eos_id: int = 3


MODEL_ARCH = {
    "transformer-base": dict(num_encoder_layer=6, num_decoder_layer=6, hidden_size=512, intermediate_size=2048, nhead=8,
                             activation_fn="relu", pre_layer_norm=True),
    "transformer-big": dict(num_encoder_layer=6, num_decoder_layer=6, hidden_size=1024, intermediate_size=4096, nhead=16,
                            activation_fn="relu", pre_layer_norm=True),
    "bert-base": dict(num_encoder_layer=12, num_decoder_layer=0, hidden_size=768, intermediate_size=3072, nhead=12,
                      activation_fn="gelu", pre_layer_norm=False),
    "bert-big": dict(num_encoder_layer=24, num_decoder_layer=0, hidden_size=1024, intermediate_size=4096, nhead=16,
                     activation_fn="gelu", pre_layer_norm=False),
    "gpt2-base": dict(num_encoder_layer=0, num_decoder_layer=12, hidden_size=768, intermediate_size=3072, nhead=12,
                      activation_fn="gelu", pre_layer_norm=True),
}


def get_config(**kwargs) -> LSModelConfig:
    """``get_config(model="transformer-base", vocab_size=..., ...)``: a preset plus overrides."""
    if "model" in kwargs:
        arch = kwargs.pop("model")
        if arch not in MODEL_ARCH:
            raise ValueError(f"{arch} architecture is not supported; one of {sorted(MODEL_ARCH)}")
        kwargs = {**MODEL_ARCH[arch], **kwargs}
    known = {f.name for f in fields(LSModelConfig)}
    unknown = set(kwargs) - known
    if unknown:
        raise TypeError(f"unknown configuration fields {sorted(unknown)}")
    return LSModelConfig(**kwargs)


class LSTransformerEncoder(nn.Module):
    def __init__(self, config: LSModelConfig, embed_tokens: LSTransformerEmbeddingLayer):
        super().__init__()
        self.config, self.embed_tokens = config, embed_tokens
        self.layers = nn.ModuleList([LSTransformerEncoderLayer(config) for _ in range(config.num_encoder_layer)])
        self.layer_norm = onn.FusedLayerNorm(config.hidden_size) if config.pre_layer_norm else None

    def forward(self, src_tokens):
        """Returns ``(encoder_out [b, s, h], padding_mask [b, s])`` (mask: True at padding)."""
        pad = src_tokens == self.config.padding_idx
        x = self.embed_tokens(src_tokens)
        mask = pad if bool(pad.any()) else None
        for layer in self.layers:
            x = layer(x, mask)
        if self.layer_norm is not None:
            x = self.layer_norm(x)
        return x, mask


class LSTransformerDecoder(nn.Module):
    def __init__(self, config: LSModelConfig, embed_tokens: LSTransformerEmbeddingLayer):
        super().__init__()
        self.config, self.embed_tokens = config, embed_tokens
        self.layers = nn.ModuleList([LSTransformerDecoderLayer(config) for _ in range(config.num_decoder_layer)])
        self.layer_norm = onn.FusedLayerNorm(config.hidden_size) if config.pre_layer_norm else None
        self.output_projection = onn.Linear(config.hidden_size, config.vocab_size, bias=False)
        self.output_projection.weight = embed_tokens.embeddings.weight  # tied

    def forward(self, trg_tokens, encoder_out, encoder_padding_mask=None, step: int = 0):
        x = self.embed_tokens(trg_tokens, step=step)
        for layer in self.layers:
            x = layer(x, encoder_out, encoder_padding_mask)
        if self.layer_norm is not None:
            x = self.layer_norm(x)
        return self.output_projection(x)


class LSTransformer(nn.Module):
    """Encoder-decoder translation model: ``forward(src_tokens, trg_tokens) -> logits [b, t, vocab]``."""

    get_config = staticmethod(get_config)

    def __init__(self, config: LSModelConfig, share_embeddings: bool = True):
        super().__init__()
        self.config = config
        enc_embed = LSTransformerEmbeddingLayer(config)
        dec_embed = enc_embed if share_embeddings else LSTransformerEmbeddingLayer(config)
        self.encoder = LSTransformerEncoder(config, enc_embed)
        self.decoder = LSTransformerDecoder(config, dec_embed)
        self.criterion = LSCrossEntropyLayer(config)

    def forward(self, src_tokens, trg_tokens, labels: Optional[torch.Tensor] = None):
        enc, mask = self.encoder(src_tokens)
        logits = self.decoder(trg_tokens, enc, mask)
        if labels is None:
            return logits
        loss, nll = self.criterion(logits, labels)
        ntok = (labels != self.config.padding_idx).sum().clamp(min=1)
        return loss / ntok, logits

    @torch.no_grad()
    def infer(self, src_tokens, max_new_tokens: int = 64, beam_size: int = 1, length_penalty: float = 0.6):
        """Greedy (``beam_size = 1``) or beam-search translation; returns ``[b, <= max_new_tokens + 1]`` token ids that
        start with ``bos_id`` and are padded after ``eos_id``."""
        cfg = self.config
        enc, mask = self.encoder(src_tokens)
        b = src_tokens.shape[0]
        if beam_size > 1:
            enc = enc.repeat_interleave(beam_size, dim=0)
            mask = mask.repeat_interleave(beam_size, dim=0) if mask is not None else None
        n = enc.shape[0]
        out = torch.full((n, 1), cfg.bos_id, dtype=torch.long, device=src_tokens.device)
        scores = torch.zeros(b, beam_size, device=src_tokens.device)
        if beam_size > 1:
            scores[:, 1:] = -1e9  # all beams start identical: only the first may spawn children at step 0
        done = torch.zeros(n, dtype=torch.bool, device=src_tokens.device)
        for _ in range(max_new_tokens):
            logp = torch.log_softmax(self.decoder(out, enc, mask)[:, -1].float(), dim=-1)
            logp[done] = -1e9
            logp[done, cfg.padding_idx] = 0.0  # finished hypotheses only extend with padding, at no cost
            if beam_size == 1:
                nxt = logp.argmax(-1)
            else:
                v = logp.shape[-1]
                cand = (scores.view(-1, 1) + logp).view(b, beam_size * v)
                scores, idx = cand.topk(beam_size, dim=-1)
                parent = idx // v + torch.arange(b, device=idx.device).unsqueeze(1) * beam_size
                nxt = (idx % v).view(-1)
                out, done = out[parent.view(-1)], done[parent.view(-1)]
            out = torch.cat([out, nxt[:, None]], dim=1)
            done = done | (nxt == cfg.eos_id)
            if bool(done.all()):
                break
        if beam_size > 1:
            lengths = (out != cfg.padding_idx).sum(-1).view(b, beam_size).float()
            best = (scores / lengths.pow(length_penalty)).argmax(-1)
            out = out.view(b, beam_size, -1)[torch.arange(b, device=out.device), best]
        return out


class LSGpt(nn.Module):
    """Decoder-only language model on :class:`LSGptEncoderLayer` blocks; ``forward(input_ids, labels=None)``."""

    get_config = staticmethod(get_config)

    def __init__(self, config: LSModelConfig):
        super().__init__()
        self.config = config
        self.embed_tokens = LSTransformerEmbeddingLayer(config)
        self.layers = nn.ModuleList([LSGptEncoderLayer(config) for _ in range(config.num_decoder_layer)])
        self.layer_norm = onn.FusedLayerNorm(config.hidden_size)
        self.lm_head = onn.Linear(config.hidden_size, config.vocab_size, bias=False)
        self.lm_head.weight = self.embed_tokens.embeddings.weight
        self.criterion = LSCrossEntropyLayer(config)

    def forward(self, input_ids, labels: Optional[torch.Tensor] = None, **unused):
        from oslo_b200.models.modeling_utils import CausalLMOutput
        from oslo_b200.ops.attention import decode_offset

        x = self.embed_tokens(input_ids, step=decode_offset())
        for layer in self.layers:
            x = layer(x)
        logits = self.lm_head(self.layer_norm(x))
        loss = None
        if labels is not None:
            shifted = torch.full_like(labels, self.config.padding_idx)
            shifted[:, :-1] = labels[:, 1:]
            total, _ = self.criterion(logits, shifted)
            loss = total / (shifted != self.config.padding_idx).sum().clamp(min=1)
        return CausalLMOutput(loss=loss, logits=logits)

    @torch.no_grad()
    def infer(self, input_ids, **kw):
        from .inference import generate

        return generate(self, input_ids, **kw)


class LSBert(nn.Module):
    """Bidirectional encoder with a first-token classification head."""

    get_config = staticmethod(get_config)

    def __init__(self, config: LSModelConfig):
        super().__init__()
        self.config = config
        self.encoder = LSTransformerEncoder(config, LSTransformerEmbeddingLayer(config))
        self.classifier = onn.Linear(config.hidden_size, config.num_labels)

    def forward(self, input_ids, labels: Optional[torch.Tensor] = None):
        x, _ = self.encoder(input_ids)
        logits = self.classifier(torch.tanh(x[:, 0]))
        if labels is None:
            return logits
        return torch.nn.functional.cross_entropy(logits.float(), labels), logits


class LSBertCrf(nn.Module):
    """Sequence tagger: bidirectional encoder -> per-token emission scores -> linear-chain CRF (the reference's
    ``BertCrf`` lsflow model, oslo/lightseq2/csrc/models/bert_crf.cc).  ``forward(input_ids, tags)`` returns the mean
    negative log-likelihood per sequence, ``infer(input_ids)`` the Viterbi paths (one list of tags per sequence, padding
    excluded)."""

    get_config = staticmethod(get_config)

    def __init__(self, config: LSModelConfig):
        super().__init__()
        from .crf import LSCRFLayer

        self.config = config
        self.encoder = LSTransformerEncoder(config, LSTransformerEmbeddingLayer(config))
        self.emission = onn.Linear(config.hidden_size, config.num_labels)
        self.crf = LSCRFLayer(config.num_labels)

    def emissions(self, input_ids):
        x, mask = self.encoder(input_ids)
        return self.emission(x), (None if mask is None else ~mask)

    def forward(self, input_ids, tags: Optional[torch.Tensor] = None):
        em, keep = self.emissions(input_ids)
        if tags is None:
            return em
        return self.crf(em, tags, keep, reduction="mean"), em

    @torch.no_grad()
    def infer(self, input_ids):
        em, keep = self.emissions(input_ids)
        return self.crf.decode(em, keep)


class LSVit(nn.Module):
    """Vision Transformer classifier on the same encoder layers: non-overlapping ``patch x patch`` patches projected by one
    linear map (a strided convolution written as unfold + GEMM, so it runs on the tcgen05 kernel), a class token, learned
    positions, pre-LayerNorm encoder, final LayerNorm, linear head on the class token (the reference's ``Vit`` inference
    model, oslo/lightseq2/inference/model/vit_encoder.cc.cu)."""

    get_config = staticmethod(get_config)

    def __init__(self, config: LSModelConfig, image_size: int = 224, patch_size: int = 16, channels: int = 3):
        super().__init__()
        if image_size % patch_size:
            raise ValueError("image_size must be a multiple of patch_size")
        if not config.pre_layer_norm:
            raise ValueError("the vision transformer is pre-LayerNorm")
        self.config, self.image_size, self.patch_size, self.channels = config, image_size, patch_size, channels
        self.num_patches = (image_size // patch_size) ** 2
        h = config.hidden_size
        self.patch_proj = onn.Linear(channels * patch_size * patch_size, h)
        self.cls_token = nn.Parameter(torch.zeros(1, 1, h))
        self.pos_embed = nn.Parameter(torch.zeros(1, self.num_patches + 1, h))
        nn.init.trunc_normal_(self.pos_embed, std=0.02)
        nn.init.trunc_normal_(self.cls_token, std=0.02)
        self.layers = nn.ModuleList([LSTransformerEncoderLayer(config) for _ in range(config.num_encoder_layer)])
        self.layer_norm = onn.FusedLayerNorm(h)
        self.classifier = onn.Linear(h, config.num_labels)

    def patches(self, pixels: torch.Tensor) -> torch.Tensor:
        """``[b, c, H, W] -> [b, patches, c * p * p]`` (channel-major inside a patch, like a Conv2d weight flattened)."""
        b, c, hh, ww = pixels.shape
        p = self.patch_size
        if (c, hh, ww) != (self.channels, self.image_size, self.image_size):
            raise ValueError(f"expected images of {self.channels} x {self.image_size} x {self.image_size}")
        x = pixels.view(b, c, hh // p, p, ww // p, p).permute(0, 2, 4, 1, 3, 5)
        return x.reshape(b, self.num_patches, c * p * p)

    def embed(self, pixels: torch.Tensor) -> torch.Tensor:
        x = self.patch_proj(self.patches(pixels).to(self.patch_proj.weight.dtype))
        x = torch.cat([self.cls_token.expand(x.shape[0], -1, -1).to(x.dtype), x], dim=1)
        return x + self.pos_embed.to(x.dtype)

    def forward(self, pixels, labels: Optional[torch.Tensor] = None):
        x = self.embed(pixels)
        for layer in self.layers:
            x = layer(x)
        logits = self.classifier(self.layer_norm(x)[:, 0])
        if labels is None:
            return logits
        return torch.nn.functional.cross_entropy(logits.float(), labels), logits


__all__ = ["LSVit", "LSBertCrf", "LSModelConfig", "MODEL_ARCH", "get_config", "LSTransformer", "LSTransformerEncoder", "LSTransformerDecoder",
           "LSGpt", "LSBert"]
