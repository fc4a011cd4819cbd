"""Transformer building blocks with the LightSeq layer interface, running on this repository's kernels.

``LSMultiheadAttentionLayer``, ``LSTransformerEncoderLayer``, ``LSTransformerDecoderLayer``, ``LSGptEncoderLayer``,
``LSTransformerEmbeddingLayer`` and ``LSCrossEntropyLayer`` mirror the modules of
oslo/lightseq2/training/ops/pytorch/*.py: they are configured through a ``get_config(...)`` object, take
``[batch, seq, hidden]`` activations plus a padding mask, support pre- and post-LayerNorm, and fuse
bias+activation+dropout and bias+dropout+residual.  Where LightSeq drives cuBLAS and its own SIMT kernels through a
layer-id registry of flat parameter buffers, these are ordinary ``nn.Module``s on the tcgen05 GEMM and the fused
norm / softmax / elementwise kernels of ``oslo_b200.ops``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

import oslo_b200.nn as onn
from oslo_b200.nn import functional as OF


@dataclass
class LSLayerConfig:
    max_batch_tokens: int = 4096
    max_seq_len: int = 512
    hidden_size: int = 512
    intermediate_size: int = 2048
    nhead: int = 8
    attn_prob_dropout_ratio: float = 0.0
    activation_dropout_ratio: float = 0.0
    hidden_dropout_ratio: float = 0.0
    pre_layer_norm: bool = True
    activation_fn: str = "gelu"
    fp16: bool = False
    local_rank: int = 0
    vocab_size: int = 0
    padding_idx: int = 0
    epsilon: float = 0.0  # label smoothing of the cross-entropy layer


def _act(name):
    return {"relu": F.relu, "gelu": lambda x: F.gelu(x, approximate="tanh")}[name]


class LSMultiheadAttentionLayer(nn.Module):
    """(pre-LN) -> fused QKV projection -> attention -> output projection -> bias + dropout + residual (-> post-LN)."""

    @staticmethod
    def get_config(**kwargs) -> LSLayerConfig:
        return LSLayerConfig(**kwargs)

    def __init__(self, config: LSLayerConfig, causal: bool = False):
        super().__init__()
        self.config, self.causal = config, causal
        h = config.hidden_size
        self.head_dim = h // config.nhead
        self.qkv = onn.Linear(h, 3 * h)
        self.out = onn.Linear(h, h, skip_bias_add=True)
        self.norm = onn.FusedLayerNorm(h)

    def forward(self, hidden_states, key_padding_mask: Optional[torch.Tensor] = None):
        cfg = self.config
        x = self.norm(hidden_states) if cfg.pre_layer_norm else hidden_states
        qkv = self.qkv(x)
        mask = None
        if key_padding_mask is not None:  # [b, s], True / 1 = padding
            mask = key_padding_mask.to(torch.float32)[:, None, None, :] * -1e4
        ctx = OF.qkv_attention(qkv, cfg.nhead, self.head_dim, layout="3hd", causal=self.causal, mask=mask)
        out, bias = self.out(ctx)
        y = OF.bias_dropout_add(out, bias, hidden_states, cfg.hidden_dropout_ratio, self.training)
        return y if cfg.pre_layer_norm else self.norm(y)


class _FeedForward(nn.Module):
    def __init__(self, config: LSLayerConfig):
        super().__init__()
        self.config = config
        self.fc1 = onn.Linear(config.hidden_size, config.intermediate_size, skip_bias_add=True)
        self.fc2 = onn.Linear(config.intermediate_size, config.hidden_size, skip_bias_add=True)
        self.norm = onn.FusedLayerNorm(config.hidden_size)

    def forward(self, hidden_states):
        cfg = self.config
        x = self.norm(hidden_states) if cfg.pre_layer_norm else hidden_states
        h, b1 = self.fc1(x)
        h = OF.bias_gelu(h, b1) if cfg.activation_fn == "gelu" else F.relu(h + b1)
        if cfg.activation_dropout_ratio and self.training:
            h = F.dropout(h, cfg.activation_dropout_ratio)
        out, b2 = self.fc2(h)
        y = OF.bias_dropout_add(out, b2, hidden_states, cfg.hidden_dropout_ratio, self.training)
        return y if cfg.pre_layer_norm else self.norm(y)


class LSTransformerEncoderLayer(nn.Module):
    get_config = staticmethod(LSMultiheadAttentionLayer.get_config)

    def __init__(self, config: LSLayerConfig, causal: bool = False):
        super().__init__()
        self.attn = LSMultiheadAttentionLayer(config, causal=causal)
        self.ffn = _FeedForward(config)

    def forward(self, hidden_states, encoder_padding_mask=None):
        return self.ffn(self.attn(hidden_states, encoder_padding_mask))


class LSGptEncoderLayer(LSTransformerEncoderLayer):
    """Decoder-only (causal) block."""

    def __init__(self, config: LSLayerConfig):
        super().__init__(config, causal=True)


class _CrossAttention(nn.Module):
    def __init__(self, config: LSLayerConfig):
        super().__init__()
        self.config = config
        h = config.hidden_size
        self.head_dim = h // config.nhead
        self.q = onn.Linear(h, h)
        self.kv = onn.Linear(h, 2 * h)
        self.out = onn.Linear(h, h, skip_bias_add=True)
        self.norm = onn.FusedLayerNorm(h)

    def forward(self, hidden_states, encoder_out, encoder_padding_mask=None):
        cfg = self.config
        x = self.norm(hidden_states) if cfg.pre_layer_norm else hidden_states
        b, t, h = x.shape
        s = encoder_out.shape[1]
        q = self.q(x).view(b, t, cfg.nhead, self.head_dim).permute(0, 2, 1, 3)
        kv = self.kv(encoder_out).view(b, s, 2, cfg.nhead, self.head_dim)
        k, v = kv[:, :, 0].permute(0, 2, 1, 3), kv[:, :, 1].permute(0, 2, 1, 3)
        scores = torch.matmul(q, k.transpose(-1, -2))
        mask = None
        if encoder_padding_mask is not None:
            mask = encoder_padding_mask.to(torch.float32)[:, None, None, :] * -1e4
        probs = OF.scale_mask_softmax(scores, 1.0 / math.sqrt(self.head_dim), False, mask)
        ctx = torch.matmul(probs, v).permute(0, 2, 1, 3).reshape(b, t, h)
        out, bias = self.out(ctx)
        y = OF.bias_dropout_add(out, bias, hidden_states, cfg.hidden_dropout_ratio, self.training)
        return y if cfg.pre_layer_norm else self.norm(y)


class LSTransformerDecoderLayer(nn.Module):
    get_config = staticmethod(LSMultiheadAttentionLayer.get_config)

    def __init__(self, config: LSLayerConfig):
        super().__init__()
        self.self_attn = LSMultiheadAttentionLayer(config, causal=True)
        self.cross_attn = _CrossAttention(config)
        self.ffn = _FeedForward(config)

    def forward(self, decoder_states, encoder_out, encoder_padding_mask=None):
        x = self.self_attn(decoder_states)
        x = self.cross_attn(x, encoder_out, encoder_padding_mask)
        return self.ffn(x)


class LSTransformerEmbeddingLayer(nn.Module):
    """Token lookup x sqrt(d) + sinusoidal positions + dropout; padding rows are zero."""

    get_config = staticmethod(LSMultiheadAttentionLayer.get_config)

    def __init__(self, config: LSLayerConfig):
        super().__init__()
        self.config = config
        self.embeddings = nn.Embedding(config.vocab_size, config.hidden_size, padding_idx=config.padding_idx)
        nn.init.normal_(self.embeddings.weight, std=config.hidden_size ** -0.5)
        pos = torch.arange(config.max_seq_len).unsqueeze(1)
        half = config.hidden_size // 2
        freq = torch.exp(torch.arange(half) * -(math.log(10000.0) / max(1, half - 1)))
        table = torch.cat([torch.sin(pos * freq), torch.cos(pos * freq)], dim=1)
        self.register_buffer("pos_embeddings", table, persistent=False)

    def forward(self, input_ids, step: int = 0):
        from .kernels import ls_embedding

        w = self.embeddings.weight
        pos = self.pos_embeddings
        if pos.dtype != w.dtype or pos.device != w.device:
            pos = self.pos_embeddings = pos.to(device=w.device, dtype=w.dtype)
        # lookup x sqrt(d) + positions + dropout with padding rows zeroed: one kernel on CUDA
        return ls_embedding(input_ids, w, pos, step, self.config.padding_idx, math.sqrt(self.config.hidden_size),
                            self.config.hidden_dropout_ratio, self.training)


class LSCrossEntropyLayer(nn.Module):
    """Label-smoothed cross-entropy; returns ``(loss_sum, nll_sum)`` over non-padding tokens like LightSeq's layer."""

    get_config = staticmethod(LSMultiheadAttentionLayer.get_config)

    def __init__(self, config: LSLayerConfig):
        super().__init__()
        self.config = config

    def forward(self, logits, targets):
        cfg = self.config
        lp = F.log_softmax(logits.float().view(-1, logits.shape[-1]), dim=-1)
        t = targets.reshape(-1)
        keep = t != cfg.padding_idx
        nll = -lp.gather(1, t.clamp(min=0).unsqueeze(1)).squeeze(1)
        smooth = -lp.mean(dim=-1)
        loss = (1.0 - cfg.epsilon) * nll + cfg.epsilon * smooth
        return (loss * keep).sum(), (nll * keep).sum()


from oslo_b200.optim import FusedAdam as LSAdam  # noqa: E402,F401
