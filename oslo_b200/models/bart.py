"""BART and mBART encoder-decoders (learned positions with offset 2; BART is post-LayerNorm, mBART pre-LayerNorm with a
final LayerNorm on each stack).

Names follow Hugging Face ``Bart*`` / ``MBart*`` (``model.encoder.layers.N.self_attn.q_proj`` ...), so their checkpoints
and the built-in tensor-parallel table (``q_proj / k_proj / v_proj / fc1`` column, ``out_proj / fc2`` row, ``embed_dim`` /
``num_heads`` divided) apply.  Cross-attention and masked self-attention run through the masked softmax path; unmasked
encoder self-attention and the causal decoder self-attention use the tcgen05 attention kernel.

Parity: oslo/transformers/models/bart/modeling_bart.py, mbart/modeling_mbart.py.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

import oslo_b200.nn as onn
from oslo_b200.nn import functional as OF

from .config import BartConfig, MBartConfig
from .heads import classification_loss, qa_loss
from .losses import token_lm_loss
from .modeling_utils import ModelOutput, PreTrainedModel, additive_mask
from .modeling_utils import active_seq2seq_cache, offset_causal_mask, seq2seq_generate


def shift_tokens_right(input_ids, pad_token_id: int, decoder_start_token_id: int):
    """Decoder inputs from labels: prepend the start token, drop the last token, turn ``-100`` into padding."""
    out = input_ids.new_zeros(input_ids.shape)
    out[:, 1:] = input_ids[:, :-1]
    out[:, 0] = decoder_start_token_id
    return out.masked_fill(out == -100, pad_token_id)


def shift_tokens_right_mbart(input_ids, pad_token_id: int):
    """mBART wraps the last non-padding token (the language id) around to the front."""
    prev = input_ids.clone().masked_fill(input_ids == -100, pad_token_id)
    last = (prev.ne(pad_token_id).sum(dim=1) - 1).unsqueeze(-1)
    start = prev.gather(1, last).squeeze(-1)
    prev[:, 1:] = prev[:, :-1].clone()
    prev[:, 0] = start
    return prev


class BartLearnedPositionalEmbedding(nn.Embedding):
    def __init__(self, num_embeddings, embedding_dim):
        super().__init__(num_embeddings + 2, embedding_dim)

    def forward(self, seq_len: int, device, past: int = 0):
        return super().forward(torch.arange(past, past + seq_len, device=device).unsqueeze(0) + 2)


class BartAttention(nn.Module):
    def __init__(self, embed_dim, num_heads, is_causal=False):
        super().__init__()
        self.embed_dim, self.num_heads = embed_dim, num_heads
        self.head_dim = embed_dim // num_heads
        self.is_causal = is_causal
        self.q_proj = onn.Linear(embed_dim, embed_dim)
        self.k_proj = onn.Linear(embed_dim, embed_dim)
        self.v_proj = onn.Linear(embed_dim, embed_dim)
        self.out_proj = onn.Linear(embed_dim, embed_dim, skip_bias_add=True)

    def forward(self, hidden_states, key_value_states=None, mask=None):
        b, t, _ = hidden_states.shape
        src = hidden_states if key_value_states is None else key_value_states
        q = self.q_proj(hidden_states).unflatten(-1, (-1, self.head_dim))
        project = lambda: (self.k_proj(src).unflatten(-1, (-1, self.head_dim)),  # noqa: E731
                           self.v_proj(src).unflatten(-1, (-1, self.head_dim)))
        cross = key_value_states is not None
        cache = active_seq2seq_cache() if (cross or self.is_causal) else None  # decoder modules only
        causal = self.is_causal and not cross
        if cache is None:
            k, v = project()
        elif cross:
            k, v = cache.cross(id(self), project)  # the encoder memory is projected on the first step only
        else:
            k, v = cache.self_append(id(self), *project())
            if cache.offset > 0:  # new tokens against stored ones: the triangle is offset, not square
                causal = False
                tri = offset_causal_mask(t, cache.offset, q.device)
                if tri is not None:
                    mask = tri if mask is None else mask + tri
        return self.out_proj(OF.attention(q, k, v, causal=causal, mask=mask))


class BartEncoderLayer(nn.Module):
    pre_norm = False

    def __init__(self, config):
        super().__init__()
        d = config.d_model
        self.self_attn = BartAttention(d, config.encoder_attention_heads)
        self.self_attn_layer_norm = onn.FusedLayerNorm(d)
        self.fc1 = onn.Linear(d, config.encoder_ffn_dim, skip_bias_add=True)
        self.fc2 = onn.Linear(config.encoder_ffn_dim, d, skip_bias_add=True)
        self.final_layer_norm = onn.FusedLayerNorm(d)
        self.act, self.p = config.activation_function, config.dropout

    def _ffn(self, x):
        h, bias = self.fc1(x)
        return self.fc2(OF.bias_act(h, bias, self.act))

    def forward(self, x, mask=None):
        a, a_bias = self.self_attn(self.self_attn_layer_norm(x) if self.pre_norm else x, mask=mask)
        x = OF.bias_dropout_add(a, a_bias, x, self.p, self.training)
        if not self.pre_norm:
            x = self.self_attn_layer_norm(x)
        f, f_bias = self._ffn(self.final_layer_norm(x) if self.pre_norm else x)
        x = OF.bias_dropout_add(f, f_bias, x, self.p, self.training)
        return x if self.pre_norm else self.final_layer_norm(x)


class BartDecoderLayer(nn.Module):
    pre_norm = False

    def __init__(self, config):
        super().__init__()
        d = config.d_model
        self.self_attn = BartAttention(d, config.decoder_attention_heads, is_causal=True)
        self.self_attn_layer_norm = onn.FusedLayerNorm(d)
        self.encoder_attn = BartAttention(d, config.decoder_attention_heads)
        self.encoder_attn_layer_norm = onn.FusedLayerNorm(d)
        self.fc1 = onn.Linear(d, config.decoder_ffn_dim, skip_bias_add=True)
        self.fc2 = onn.Linear(config.decoder_ffn_dim, d, skip_bias_add=True)
        self.final_layer_norm = onn.FusedLayerNorm(d)
        self.act, self.p = config.activation_function, config.dropout

    _ffn = BartEncoderLayer._ffn

    def forward(self, x, self_mask=None, encoder_hidden_states=None, cross_mask=None):
        a, a_bias = self.self_attn(self.self_attn_layer_norm(x) if self.pre_norm else x, mask=self_mask)
        x = OF.bias_dropout_add(a, a_bias, x, self.p, self.training)
        if not self.pre_norm:
            x = self.self_attn_layer_norm(x)
        if encoder_hidden_states is not None:
            c, c_bias = self.encoder_attn(self.encoder_attn_layer_norm(x) if self.pre_norm else x, encoder_hidden_states, cross_mask)
            x = OF.bias_dropout_add(c, c_bias, x, self.p, self.training)
            if not self.pre_norm:
                x = self.encoder_attn_layer_norm(x)
        f, f_bias = self._ffn(self.final_layer_norm(x) if self.pre_norm else x)
        x = OF.bias_dropout_add(f, f_bias, x, self.p, self.training)
        return x if self.pre_norm else self.final_layer_norm(x)


class BartEncoder(nn.Module):
    layer_cls, final_norm = BartEncoderLayer, False

    def __init__(self, config, embed_tokens):
        super().__init__()
        d = config.d_model
        self.embed_scale = math.sqrt(d) if config.scale_embedding else 1.0
        self.embed_tokens = embed_tokens
        self.embed_positions = BartLearnedPositionalEmbedding(config.max_position_embeddings, d)
        self.layers = nn.ModuleList([self.layer_cls(config) for _ in range(config.encoder_layers)])
        self.layernorm_embedding = onn.FusedLayerNorm(d)
        if self.final_norm:
            self.layer_norm = onn.FusedLayerNorm(d)
        self.dropout = nn.Dropout(config.dropout)
        self.gradient_checkpointing = False

    def forward(self, input_ids, attention_mask=None):
        x = self.embed_tokens(input_ids) * self.embed_scale + self.embed_positions(input_ids.shape[1], input_ids.device)
        x = self.dropout(self.layernorm_embedding(x))
        mask = additive_mask(attention_mask, torch.float32)
        for layer in self.layers:
            if self.gradient_checkpointing and self.training:
                x = torch.utils.checkpoint.checkpoint(layer, x, mask, use_reentrant=False)
            else:
                x = layer(x, mask)
        return self.layer_norm(x) if self.final_norm else x


def causal_additive_mask(attention_mask, tgt_len, dtype=torch.float32):
    """Padding mask of the decoder inputs combined with the causal triangle, additive ``[b, 1, t, t]``."""
    pad = additive_mask(attention_mask, dtype, tgt_len)
    tri = torch.full((tgt_len, tgt_len), torch.finfo(dtype).min, device=attention_mask.device).triu(1)
    return (pad + tri).clamp_min(torch.finfo(dtype).min)


class BartDecoder(nn.Module):
    layer_cls, final_norm = BartDecoderLayer, False

    def __init__(self, config, embed_tokens):
        super().__init__()
        d = config.d_model
        self.embed_scale = math.sqrt(d) if config.scale_embedding else 1.0
        self.embed_tokens = embed_tokens
        self.embed_positions = BartLearnedPositionalEmbedding(config.max_position_embeddings, d)
        self.layers = nn.ModuleList([self.layer_cls(config) for _ in range(config.decoder_layers)])
        self.layernorm_embedding = onn.FusedLayerNorm(d)
        if self.final_norm:
            self.layer_norm = onn.FusedLayerNorm(d)
        self.dropout = nn.Dropout(config.dropout)
        self.gradient_checkpointing = False

    def forward(self, input_ids, attention_mask=None, encoder_hidden_states=None, encoder_attention_mask=None):
        t = input_ids.shape[1]
        cache = active_seq2seq_cache()
        past = cache.offset if cache is not None else 0
        x = self.embed_tokens(input_ids) * self.embed_scale + self.embed_positions(t, input_ids.device, past)
        x = self.dropout(self.layernorm_embedding(x))
        self_mask = causal_additive_mask(attention_mask, t) if attention_mask is not None else None
        cross_mask = additive_mask(encoder_attention_mask, torch.float32)
        for layer in self.layers:
            if self.gradient_checkpointing and self.training:
                x = torch.utils.checkpoint.checkpoint(layer, x, self_mask, encoder_hidden_states, cross_mask, use_reentrant=False)
            else:
                x = layer(x, self_mask, encoder_hidden_states, cross_mask)
        return self.layer_norm(x) if self.final_norm else x


class BartPreTrainedModel(PreTrainedModel):
    config_class = BartConfig
    base_model_prefix = "model"
    encoder_cls, decoder_cls = BartEncoder, BartDecoder

    def get_input_embeddings(self):
        return getattr(self, "model", self).shared

    def gradient_checkpointing_enable(self):
        m = getattr(self, "model", self)
        for part in (getattr(m, "encoder", None), getattr(m, "decoder", None)):
            if part is not None:
                part.gradient_checkpointing = True

    def _shift(self, labels):
        return shift_tokens_right(labels, self.config.pad_token_id, self.config.decoder_start_token_id)


class BartModel(BartPreTrainedModel):
    def __init__(self, config):
        super().__init__(config)
        self.shared = nn.Embedding(config.vocab_size, config.d_model, padding_idx=config.pad_token_id)
        self.encoder = self.encoder_cls(config, self.shared)
        self.decoder = self.decoder_cls(config, self.shared)
        self.post_init()

    def forward(self, input_ids=None, attention_mask=None, decoder_input_ids=None, decoder_attention_mask=None,
                encoder_outputs=None, **unused):
        if decoder_input_ids is None:
            decoder_input_ids = self._shift(input_ids)
        enc = encoder_outputs if encoder_outputs is not None else self.encoder(input_ids, attention_mask)
        dec = self.decoder(decoder_input_ids, decoder_attention_mask, enc, attention_mask)
        return ModelOutput(last_hidden_state=dec, encoder_last_hidden_state=enc)


class BartForConditionalGeneration(BartPreTrainedModel):
    model_cls = BartModel

    def __init__(self, config):
        super().__init__(config)
        self.model = self.model_cls(config)
        self.register_buffer("final_logits_bias", torch.zeros((1, config.vocab_size)))
        self.lm_head = onn.Linear(config.d_model, config.vocab_size, bias=False)
        self.post_init()

    def get_output_embeddings(self):
        return self.lm_head

    def get_encoder(self):
        return self.model.encoder

    def forward(self, input_ids=None, attention_mask=None, decoder_input_ids=None, decoder_attention_mask=None, labels=None,
                encoder_outputs=None, **unused):
        if labels is not None and decoder_input_ids is None:
            decoder_input_ids = self._shift(labels)
        out = self.model(input_ids, attention_mask, decoder_input_ids, decoder_attention_mask, encoder_outputs)
        logits = self.lm_head(out.last_hidden_state)
        if self.final_logits_bias.shape[-1] == logits.shape[-1] and bool(self.final_logits_bias.any()):
            logits = logits + self.final_logits_bias.to(logits.dtype)
        loss = None
        if labels is not None:
            res = token_lm_loss(self, logits, labels)
            loss, logits = res.value, (None if res.consumed_logits else logits)
        return ModelOutput(loss=loss, logits=logits, encoder_last_hidden_state=out.encoder_last_hidden_state)

    def pipeline_units(self):
        """Encoder embedding, one unit per encoder layer, the hand-over (encoder output norm + decoder embedding), one unit
        per decoder layer, head + loss.  One activation crosses a stage boundary, so from the hand-over on it is the encoder
        output and the decoder state concatenated along the sequence (``[b, s_enc + s_dec, d]``): every decoder unit splits it,
        runs its layer with the encoder part as memory and joins it again, and the gradient of both parts flows back through
        the same tensor."""
        from oslo_b200.parallel.pipeline_parallel.partitioner import PipeUnit

        enc, dec = self.model.encoder, self.model.decoder

        def dec_ids(state):
            ids = state.get("decoder_input_ids")
            return ids if ids is not None else self._shift(state["labels"] if state.get("labels") is not None else state["input_ids"])

        def enc_embed(state):
            ids = state["input_ids"]
            x = enc.embed_tokens(ids) * enc.embed_scale + enc.embed_positions(ids.shape[1], ids.device)
            state["hidden"] = enc.dropout(enc.layernorm_embedding(x))
            return state

        def make_enc(layer):
            def run(state):
                state["hidden"] = layer(state["hidden"], additive_mask(state.get("attention_mask"), torch.float32))
                return state

            return run

        def hand_over(state):
            memory = enc.layer_norm(state["hidden"]) if enc.final_norm else state["hidden"]
            ids = dec_ids(state)
            y = dec.embed_tokens(ids) * dec.embed_scale + dec.embed_positions(ids.shape[1], ids.device)
            y = dec.dropout(dec.layernorm_embedding(y))
            state["hidden"] = torch.cat([memory, y], dim=1)
            return state

        def make_dec(layer):
            def run(state):
                s_enc = state["input_ids"].shape[1]
                memory, y = state["hidden"][:, :s_enc], state["hidden"][:, s_enc:]
                dmask = state.get("decoder_attention_mask")
                self_mask = causal_additive_mask(dmask, y.shape[1]) if dmask is not None else None
                y = layer(y, self_mask, memory, additive_mask(state.get("attention_mask"), torch.float32))
                state["hidden"] = torch.cat([memory, y], dim=1)
                return state

            return run

        def head(state):
            y = state["hidden"][:, state["input_ids"].shape[1]:]
            if dec.final_norm:
                y = dec.layer_norm(y)
            logits = self.lm_head(y)
            if self.final_logits_bias.shape[-1] == logits.shape[-1] and bool(self.final_logits_bias.any()):
                logits = logits + self.final_logits_bias.to(logits.dtype)
            state["logits"] = logits
            if state.get("labels") is not None:
                res = token_lm_loss(self, logits, state["labels"])
                state["loss"] = res.value
                if res.consumed_logits:
                    state["logits"] = None
            return state

        shared = self.model.shared
        units = [PipeUnit("encoder.embed", [shared, enc.embed_positions, enc.layernorm_embedding], enc_embed)]
        units += [PipeUnit(f"encoder.layers.{i}", [l], make_enc(l)) for i, l in enumerate(enc.layers)]
        units.append(PipeUnit("decoder.embed", ([enc.layer_norm] if enc.final_norm else [])
                              + [shared, dec.embed_positions, dec.layernorm_embedding], hand_over))
        units += [PipeUnit(f"decoder.layers.{i}", [l], make_dec(l)) for i, l in enumerate(dec.layers)]
        units.append(PipeUnit("head", ([dec.layer_norm] if dec.final_norm else []) + [self.lm_head], head))
        return units

    @torch.no_grad()
    def generate(self, input_ids, attention_mask=None, max_new_tokens: int = 32, num_beams: int = 1, length_penalty: float = 1.0,
                 use_cache: bool = True):
        """Greedy (``num_beams = 1``) or beam-search decoding.  The encoder runs once; with ``use_cache`` every step feeds
        the newest target token only and the attention modules keep their keys / values (``Seq2SeqCache``)."""
        cfg = self.config
        return seq2seq_generate(
            self, lambda ids, mask: self.model.encoder(ids, mask),
            lambda enc, mask, dec: self.forward(attention_mask=mask, decoder_input_ids=dec, encoder_outputs=enc).logits[:, -1],
            input_ids, attention_mask, max_new_tokens, num_beams, length_penalty, cfg.decoder_start_token_id, cfg.eos_token_id,
            cfg.pad_token_id, use_cache)


class BartClassificationHead(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = onn.Linear(config.d_model, config.d_model)
        self.dropout = nn.Dropout(config.classifier_dropout)
        self.out_proj = onn.Linear(config.d_model, config.num_labels)

    def forward(self, x):
        return self.out_proj(self.dropout(torch.tanh(self.dense(self.dropout(x)))))


class BartForSequenceClassification(BartPreTrainedModel):
    """Classifies from the decoder state at the last ``eos`` token of every row."""

    model_cls = BartModel

    def __init__(self, config):
        super().__init__(config)
        self.model = self.model_cls(config)
        self.classification_head = BartClassificationHead(config)
        self.post_init()

    def forward(self, input_ids, attention_mask=None, decoder_input_ids=None, decoder_attention_mask=None, labels=None, **unused):
        h = self.model(input_ids, attention_mask, decoder_input_ids, decoder_attention_mask).last_hidden_state
        eos = input_ids.eq(self.config.eos_token_id)
        if len(torch.unique_consecutive(eos.sum(1))) > 1:
            raise ValueError("every row needs the same number of <eos> tokens")
        sent = h[eos, :].view(h.shape[0], -1, h.shape[-1])[:, -1, :]
        logits = self.classification_head(sent)
        return ModelOutput(loss=classification_loss(logits, labels, self.config.num_labels), logits=logits)


class BartForQuestionAnswering(BartPreTrainedModel):
    model_cls = BartModel

    def __init__(self, config):
        super().__init__(config)
        self.model = self.model_cls(config)
        self.qa_outputs = onn.Linear(config.d_model, 2)
        self.post_init()

    def forward(self, input_ids, attention_mask=None, decoder_input_ids=None, decoder_attention_mask=None,
                start_positions=None, end_positions=None, **unused):
        h = self.model(input_ids, attention_mask, decoder_input_ids, decoder_attention_mask).last_hidden_state
        start, end = (t.squeeze(-1).contiguous() for t in self.qa_outputs(h).split(1, dim=-1))
        return ModelOutput(loss=qa_loss(start, end, start_positions, end_positions), start_logits=start, end_logits=end)


class _DecoderWrapper(nn.Module):
    def __init__(self, config, decoder_cls):
        super().__init__()
        self.decoder = decoder_cls(config, nn.Embedding(config.vocab_size, config.d_model, padding_idx=config.pad_token_id))


class BartForCausalLM(BartPreTrainedModel):
    """The decoder stack alone as a left-to-right language model (``model.decoder.*`` + ``lm_head``).  As in the Hugging
    Face class, ``labels`` are compared position by position (the caller supplies already shifted labels)."""

    def __init__(self, config):
        super().__init__(config)
        self.model = _DecoderWrapper(config, self.decoder_cls)
        self.lm_head = onn.Linear(config.d_model, config.vocab_size, bias=False)
        self.post_init()

    def get_input_embeddings(self):
        return self.model.decoder.embed_tokens

    def get_output_embeddings(self):
        return self.lm_head

    def forward(self, input_ids, attention_mask=None, encoder_hidden_states=None, encoder_attention_mask=None, labels=None, **unused):
        logits = self.lm_head(self.model.decoder(input_ids, attention_mask, encoder_hidden_states, encoder_attention_mask))
        loss = None
        if labels is not None:
            res = token_lm_loss(self, logits, labels)
            loss, logits = res.value, (None if res.consumed_logits else logits)
        return ModelOutput(loss=loss, logits=logits)


# ------------------------------------------------------------------------------------------------------- mBART
class MBartEncoderLayer(BartEncoderLayer):
    pre_norm = True


class MBartDecoderLayer(BartDecoderLayer):
    pre_norm = True


class MBartEncoder(BartEncoder):
    layer_cls, final_norm = MBartEncoderLayer, True


class MBartDecoder(BartDecoder):
    layer_cls, final_norm = MBartDecoderLayer, True


class MBartPreTrainedModel(BartPreTrainedModel):
    config_class = MBartConfig
    encoder_cls, decoder_cls = MBartEncoder, MBartDecoder

    def _shift(self, labels):
        return shift_tokens_right_mbart(labels, self.config.pad_token_id)


class MBartModel(BartModel, MBartPreTrainedModel):
    pass


class MBartForConditionalGeneration(BartForConditionalGeneration, MBartPreTrainedModel):
    model_cls = MBartModel


class MBartForSequenceClassification(BartForSequenceClassification, MBartPreTrainedModel):
    model_cls = MBartModel


class MBartForQuestionAnswering(BartForQuestionAnswering, MBartPreTrainedModel):
    model_cls = MBartModel


class MBartForCausalLM(BartForCausalLM, MBartPreTrainedModel):
    pass


__all__ = [n for n in globals() if n.startswith(("Bart", "MBart")) and not n.endswith("Config")] + ["shift_tokens_right"]
