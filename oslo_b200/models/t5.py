"""T5 and mT5 encoder-decoders: RMS LayerNorm without bias, no attention scaling, bucketed relative position bias added to
the scores, ReLU or gated-GELU feed-forward without biases.

Names follow Hugging Face ``T5*`` / ``MT5*`` (``encoder.block.N.layer.0.SelfAttention.q`` ...), so their checkpoints and
the built-in tensor-parallel table (``q / k / v / wi*`` column, ``o / wo`` row, ``d_model`` / ``n_heads`` / ``inner_dim``
divided, ``relative_attention_bias`` split over heads) apply.  Every attention carries an additive bias here, so the scores
go through the masked softmax path; the norms and gated activation run on the fused kernels.

Parity: oslo/transformers/models/t5/modeling_t5.py, mt5/modeling_mt5.py.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

import oslo_b200.nn as onn
from oslo_b200.nn import functional as OF
from oslo_b200.ops.activation import act_reference

from .config import MT5Config, T5Config
from .losses import token_lm_loss
from .modeling_utils import ModelOutput, PreTrainedModel, additive_mask
from .modeling_utils import active_seq2seq_cache, offset_causal_mask, seq2seq_generate


class T5LayerNorm(onn.FusedRMSNorm):
    """Scale-only RMS normalisation (the variance is taken in fp32, no mean subtraction, no bias)."""

    def __init__(self, hidden_size, eps=1e-6):
        super().__init__(hidden_size, eps=eps)


class T5DenseActDense(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.wi = onn.Linear(config.d_model, config.d_ff, bias=False)
        self.wo = onn.Linear(config.d_ff, config.d_model, bias=False)
        self.act, self.dropout = config.dense_act_fn, nn.Dropout(config.dropout_rate)

    def forward(self, x):
        return self.wo(self.dropout(OF.bias_act(self.wi(x), None, self.act)))


class T5DenseGatedActDense(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.wi_0 = onn.Linear(config.d_model, config.d_ff, bias=False)
        self.wi_1 = onn.Linear(config.d_model, config.d_ff, bias=False)
        self.wo = onn.Linear(config.d_ff, config.d_model, bias=False)
        self.act, self.dropout = config.dense_act_fn, nn.Dropout(config.dropout_rate)

    def forward(self, x):
        return self.wo(self.dropout(OF.bias_act(self.wi_0(x), None, self.act) * self.wi_1(x)))


class T5LayerFF(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.DenseReluDense = T5DenseGatedActDense(config) if config.is_gated_act else T5DenseActDense(config)
        self.layer_norm = T5LayerNorm(config.d_model, eps=config.layer_norm_epsilon)
        self.p = config.dropout_rate

    def forward(self, x):
        return OF.bias_dropout_add(self.DenseReluDense(self.layer_norm(x)), None, x, self.p, self.training)


def relative_position_bucket(relative_position, bidirectional=True, num_buckets=32, max_distance=128):
    """Bucket index of ``key position - query position``: exact for small offsets, logarithmic up to ``max_distance``."""
    buckets = 0
    if bidirectional:
        num_buckets //= 2
        buckets = buckets + (relative_position > 0).long() * num_buckets
        relative_position = relative_position.abs()
    else:
        relative_position = -torch.min(relative_position, torch.zeros_like(relative_position))
    max_exact = num_buckets // 2
    is_small = relative_position < max_exact
    large = max_exact + (torch.log(relative_position.float() / max_exact) / math.log(max_distance / max_exact)
                         * (num_buckets - max_exact)).long()
    large = torch.min(large, torch.full_like(large, num_buckets - 1))
    return buckets + torch.where(is_small, relative_position, large)


class T5Attention(nn.Module):
    def __init__(self, config, has_relative_attention_bias=False, is_decoder=False):
        super().__init__()
        self.is_decoder = is_decoder
        self.has_relative_attention_bias = has_relative_attention_bias
        self.relative_attention_num_buckets = config.relative_attention_num_buckets
        self.relative_attention_max_distance = config.relative_attention_max_distance
        self.d_model, self.key_value_proj_dim, self.n_heads = config.d_model, config.d_kv, config.num_heads
        self.inner_dim = self.n_heads * self.key_value_proj_dim
        self.q = onn.Linear(self.d_model, self.inner_dim, bias=False)
        self.k = onn.Linear(self.d_model, self.inner_dim, bias=False)
        self.v = onn.Linear(self.d_model, self.inner_dim, bias=False)
        self.o = onn.Linear(self.inner_dim, self.d_model, bias=False)
        if has_relative_attention_bias:
            self.relative_attention_bias = nn.Embedding(self.relative_attention_num_buckets, self.n_heads)

    def compute_bias(self, q_len, k_len, device):
        ctx = torch.arange(q_len, dtype=torch.long, device=device)[:, None]
        mem = torch.arange(k_len, dtype=torch.long, device=device)[None, :]
        bucket = relative_position_bucket(mem - ctx, not self.is_decoder, self.relative_attention_num_buckets,
                                          self.relative_attention_max_distance)
        return self.relative_attention_bias(bucket).permute(2, 0, 1).unsqueeze(0)  # [1, heads, q, k]

    def forward(self, x, key_value_states=None, position_bias=None):
        b, t, _ = x.shape
        src = x if key_value_states is None else key_value_states
        hd = self.key_value_proj_dim
        q = self.q(x).unflatten(-1, (-1, hd))
        project = lambda: (self.k(src).unflatten(-1, (-1, hd)), self.v(src).unflatten(-1, (-1, hd)))  # noqa: E731
        cache = active_seq2seq_cache() if self.is_decoder else None
        if cache is None:
            k, v = project()
        elif key_value_states is None:
            k, v = cache.self_append(id(self), *project())  # keys / values of every target token so far
        else:
            k, v = cache.cross(id(self), project)  # the encoder memory is projected on the first step only
        return self.o(OF.attention(q, k, v, causal=False, scale=1.0, mask=position_bias))


class T5LayerSelfAttention(nn.Module):
    def __init__(self, config, has_relative_attention_bias=False, is_decoder=False):
        super().__init__()
        self.SelfAttention = T5Attention(config, has_relative_attention_bias, is_decoder)
        self.layer_norm = T5LayerNorm(config.d_model, eps=config.layer_norm_epsilon)
        self.p = config.dropout_rate

    def forward(self, x, position_bias):
        return OF.bias_dropout_add(self.SelfAttention(self.layer_norm(x), None, position_bias), None, x, self.p, self.training)


class T5LayerCrossAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.EncDecAttention = T5Attention(config, False, True)
        self.layer_norm = T5LayerNorm(config.d_model, eps=config.layer_norm_epsilon)
        self.p = config.dropout_rate

    def forward(self, x, encoder_hidden_states, mask):
        return OF.bias_dropout_add(self.EncDecAttention(self.layer_norm(x), encoder_hidden_states, mask), None, x, self.p,
                                   self.training)


class T5Block(nn.Module):
    def __init__(self, config, has_relative_attention_bias=False, is_decoder=False):
        super().__init__()
        self.is_decoder = is_decoder
        self.layer = nn.ModuleList([T5LayerSelfAttention(config, has_relative_attention_bias, is_decoder)])
        if is_decoder:
            self.layer.append(T5LayerCrossAttention(config))
        self.layer.append(T5LayerFF(config))

    def forward(self, x, position_bias, encoder_hidden_states=None, cross_mask=None):
        x = self.layer[0](x, position_bias)
        if self.is_decoder and encoder_hidden_states is not None:
            x = self.layer[1](x, encoder_hidden_states, cross_mask)
        return self.layer[-1](x)


class T5Stack(nn.Module):
    def __init__(self, config, embed_tokens, is_decoder=False):
        super().__init__()
        self.is_decoder = is_decoder
        self.embed_tokens = embed_tokens
        n = config.num_decoder_layers if is_decoder else config.num_layers
        self.block = nn.ModuleList([T5Block(config, has_relative_attention_bias=(i == 0), is_decoder=is_decoder) for i in range(n)])
        self.final_layer_norm = T5LayerNorm(config.d_model, eps=config.layer_norm_epsilon)
        self.dropout = nn.Dropout(config.dropout_rate)
        self.gradient_checkpointing = False

    def forward(self, input_ids, attention_mask=None, encoder_hidden_states=None, encoder_attention_mask=None):
        b, t = input_ids.shape
        x = self.dropout(self.embed_tokens(input_ids))
        cache = active_seq2seq_cache() if self.is_decoder else None
        past = cache.offset if cache is not None else 0
        bias = self.block[0].layer[0].SelfAttention.compute_bias(past + t, past + t, input_ids.device).float()[:, :, past:]
        if self.is_decoder:
            tri = offset_causal_mask(t, past, input_ids.device)
            if tri is not None:
                bias = bias + tri
        if attention_mask is not None:
            bias = bias + additive_mask(attention_mask, torch.float32)
        cross_mask = additive_mask(encoder_attention_mask, torch.float32)
        for blk in self.block:
            if self.gradient_checkpointing and self.training:
                x = torch.utils.checkpoint.checkpoint(blk, x, bias, encoder_hidden_states, cross_mask, use_reentrant=False)
            else:
                x = blk(x, bias, encoder_hidden_states, cross_mask)
        return self.dropout(self.final_layer_norm(x))


class T5PreTrainedModel(PreTrainedModel):
    config_class = T5Config
    base_model_prefix = "transformer"

    def _init_weights(self, module):
        f = self.config.initializer_factor
        d, kv, h = self.config.d_model, self.config.d_kv, self.config.num_heads
        if isinstance(module, T5LayerNorm):
            module.weight.data.fill_(f)
        elif isinstance(module, T5Attention):
            module.q.weight.data.normal_(0.0, f * (d * kv) ** -0.5)
            module.k.weight.data.normal_(0.0, f * d ** -0.5)
            module.v.weight.data.normal_(0.0, f * d ** -0.5)
            module.o.weight.data.normal_(0.0, f * (h * kv) ** -0.5)
            if module.has_relative_attention_bias:
                module.relative_attention_bias.weight.data.normal_(0.0, f * d ** -0.5)
        elif isinstance(module, (T5DenseActDense, T5DenseGatedActDense)):
            for name in ("wi", "wi_0", "wi_1"):
                if hasattr(module, name):
                    getattr(module, name).weight.data.normal_(0.0, f * d ** -0.5)
            module.wo.weight.data.normal_(0.0, f * self.config.d_ff ** -0.5)
        elif isinstance(module, nn.Embedding) and module.embedding_dim == d:
            module.weight.data.normal_(0.0, f)

    def get_input_embeddings(self):
        return self.shared

    def gradient_checkpointing_enable(self):
        for part in (getattr(self, "encoder", None), getattr(self, "decoder", None)):
            if part is not None:
                part.gradient_checkpointing = True

    def _shift_right(self, labels):
        out = labels.new_zeros(labels.shape)
        out[:, 1:] = labels[:, :-1]
        out[:, 0] = self.config.decoder_start_token_id
        return out.masked_fill(out == -100, self.config.pad_token_id)


class T5EncoderModel(T5PreTrainedModel):
    def __init__(self, config):
        super().__init__(config)
        self.shared = nn.Embedding(config.vocab_size, config.d_model)
        self.encoder = T5Stack(config, self.shared)
        self.post_init()

    def forward(self, input_ids, attention_mask=None, **unused):
        return ModelOutput(last_hidden_state=self.encoder(input_ids, attention_mask))


class T5Model(T5PreTrainedModel):
    def __init__(self, config):
        super().__init__(config)
        self.shared = nn.Embedding(config.vocab_size, config.d_model)
        self.encoder = T5Stack(config, self.shared)
        self.decoder = T5Stack(config, self.shared, is_decoder=True)
        self.post_init()

    def forward(self, input_ids=None, attention_mask=None, decoder_input_ids=None, decoder_attention_mask=None,
                encoder_outputs=None, **unused):
        enc = encoder_outputs if encoder_outputs is not None else self.encoder(input_ids, attention_mask)
        dec = self.decoder(decoder_input_ids, decoder_attention_mask, enc, attention_mask)
        return ModelOutput(last_hidden_state=dec, encoder_last_hidden_state=enc)


class T5ForConditionalGeneration(T5Model):
    def __init__(self, config):
        super().__init__(config)
        self.lm_head = onn.Linear(config.d_model, config.vocab_size, bias=False)
        self.post_init()

    def get_output_embeddings(self):
        return getattr(self, "lm_head", None)  # the base constructor runs post_init before the head exists

    def get_encoder(self):
        return self.encoder

    def forward(self, input_ids=None, attention_mask=None, decoder_input_ids=None, decoder_attention_mask=None, labels=None,
                encoder_outputs=None, **unused):
        if labels is not None and decoder_input_ids is None:
            decoder_input_ids = self._shift_right(labels)
        out = T5Model.forward(self, input_ids, attention_mask, decoder_input_ids, decoder_attention_mask, encoder_outputs)
        h = out.last_hidden_state
        if getattr(self.config, "tie_word_embeddings", True):
            h = h * (self.config.d_model ** -0.5)
        logits = self.lm_head(h)
        loss = None
        if labels is not None:
            res = token_lm_loss(self, logits, labels)
            loss, logits = res.value, (None if res.consumed_logits else logits)
        return ModelOutput(loss=loss, logits=logits, encoder_last_hidden_state=out.encoder_last_hidden_state)

    def pipeline_units(self):
        """Same plan as BART's: encoder embedding, encoder blocks, hand-over (encoder final norm + decoder embedding with the
        two activations joined along the sequence), decoder blocks, head + loss.  The relative-position bias table lives in
        the first block of each stack and is used by all of them: it is listed in every block unit, so each stage that owns
        a block keeps a copy and the copies' gradients are summed after the backward pass."""
        from oslo_b200.parallel.pipeline_parallel.partitioner import PipeUnit

        enc, dec = self.encoder, self.decoder
        enc_rel = enc.block[0].layer[0].SelfAttention
        dec_rel = dec.block[0].layer[0].SelfAttention

        def dec_ids(state):
            ids = state.get("decoder_input_ids")
            return ids if ids is not None else self._shift_right(state["labels"])

        def enc_embed(state):
            state["hidden"] = enc.dropout(enc.embed_tokens(state["input_ids"]))
            return state

        def enc_bias(state):
            s = state["input_ids"].shape[1]
            bias = enc_rel.compute_bias(s, s, state["input_ids"].device).float()
            if state.get("attention_mask") is not None:
                bias = bias + additive_mask(state["attention_mask"], torch.float32)
            return bias

        def make_enc(blk):
            def run(state):
                state["hidden"] = blk(state["hidden"], enc_bias(state))
                return state

            return run

        def hand_over(state):
            memory = enc.dropout(enc.final_layer_norm(state["hidden"]))
            y = dec.dropout(dec.embed_tokens(dec_ids(state)))
            state["hidden"] = torch.cat([memory, y], dim=1)
            return state

        def make_dec(blk):
            def run(state):
                s_enc = state["input_ids"].shape[1]
                memory, y = state["hidden"][:, :s_enc], state["hidden"][:, s_enc:]
                t = y.shape[1]
                bias = dec_rel.compute_bias(t, t, y.device).float()
                bias = bias + torch.full((t, t), torch.finfo(torch.float32).min, device=y.device).triu(1)
                if state.get("decoder_attention_mask") is not None:
                    bias = bias + additive_mask(state["decoder_attention_mask"], torch.float32)
                y = blk(y, bias, memory, additive_mask(state.get("attention_mask"), torch.float32))
                state["hidden"] = torch.cat([memory, y], dim=1)
                return state

            return run

        def head(state):
            y = dec.dropout(dec.final_layer_norm(state["hidden"][:, state["input_ids"].shape[1]:]))
            if getattr(self.config, "tie_word_embeddings", True):
                y = y * (self.config.d_model ** -0.5)
            logits = self.lm_head(y)
            state["logits"] = logits
            if state.get("labels") is not None:
                res = token_lm_loss(self, logits, state["labels"])
                state["loss"] = res.value
                if res.consumed_logits:
                    state["logits"] = None
            return state

        enc_table, dec_table = enc_rel.relative_attention_bias, dec_rel.relative_attention_bias
        units = [PipeUnit("encoder.embed", [self.shared], enc_embed)]
        units += [PipeUnit(f"encoder.block.{i}", [b, enc_table], make_enc(b)) for i, b in enumerate(enc.block)]
        units.append(PipeUnit("decoder.embed", [enc.final_layer_norm, self.shared], hand_over))
        units += [PipeUnit(f"decoder.block.{i}", [b, dec_table], make_dec(b)) for i, b in enumerate(dec.block)]
        units.append(PipeUnit("head", [dec.final_layer_norm, self.lm_head], head))
        return units

    @torch.no_grad()
    def generate(self, input_ids, attention_mask=None, max_new_tokens: int = 32, num_beams: int = 1, length_penalty: float = 1.0,
                 use_cache: bool = True):
        """Greedy (``num_beams = 1``) or beam-search decoding.  The encoder runs once; with ``use_cache`` every step feeds
        the newest target token only and the attention modules keep their keys / values (``Seq2SeqCache``)."""
        cfg = self.config
        return seq2seq_generate(
            self, lambda ids, mask: self.encoder(ids, mask),
            lambda enc, mask, dec: self.forward(attention_mask=mask, decoder_input_ids=dec, encoder_outputs=enc).logits[:, -1],
            input_ids, attention_mask, max_new_tokens, num_beams, length_penalty, cfg.decoder_start_token_id, cfg.eos_token_id,
            cfg.pad_token_id, use_cache)


class MT5PreTrainedModel(T5PreTrainedModel):
    config_class = MT5Config


class MT5EncoderModel(T5EncoderModel, MT5PreTrainedModel):
    pass


class MT5Model(T5Model, MT5PreTrainedModel):
    pass


class MT5ForConditionalGeneration(T5ForConditionalGeneration, MT5PreTrainedModel):
    pass


__all__ = [n for n in globals() if n.startswith(("T5", "MT5")) and not n.endswith("Config")]
