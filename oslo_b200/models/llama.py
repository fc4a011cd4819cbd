"""Llama style decoder (RMSNorm, rotary embedding on the whole head dim, SwiGLU MLP, no biases).

State-dict names follow Hugging Face ``LlamaForCausalLM`` (``model.layers.N.self_attn.q_proj`` ...); rotary uses the
half-rotation ("NeoX") convention as there.  Grouped-query attention is supported by repeating KV heads.
The reference has no Llama model or mapping; this file and the ``Llama`` mapping entry add them.
"""
from __future__ import annotations

import torch
import torch.nn as nn

import oslo_b200.nn as onn
from oslo_b200.nn import functional as OF
from oslo_b200.ops.activation import swiglu2

from .config import LlamaConfig
from .modeling_utils import CausalLMOutput, PreTrainedModel


class LlamaAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.head_dim = config.hidden_size // config.num_attention_heads
        self.num_heads = config.num_attention_heads
        self.num_key_value_heads = config.num_key_value_heads
        self.rope_theta = config.rope_theta
        self.max_positions = config.max_position_embeddings
        h, kv = config.hidden_size, config.num_key_value_heads * self.head_dim
        self.q_proj = onn.Linear(h, h, bias=False)
        self.k_proj = onn.Linear(h, kv, bias=False)
        self.v_proj = onn.Linear(h, kv, bias=False)
        self.o_proj = onn.Linear(h, h, bias=False)
        self._rope = None

    def _tables(self, seq, device):
        if self._rope is None or self._rope[0].shape[0] < seq or self._rope[0].device != device:
            self._rope = OF.rope_tables(max(seq, self.max_positions), self.head_dim, self.rope_theta, device)
        # rows [0, seq): the kernels take a token's position as (flattened token index) mod (table rows)
        return self._rope[0][:seq], self._rope[1][:seq]

    def forward(self, x, attention_mask=None):
        q = self.q_proj(x)
        k = self.k_proj(x)
        v = self.v_proj(x)
        b, s = q.shape[0], q.shape[1]  # from the projection: under sequence parallelism it has gathered the token shards
        hq, hkv = q.shape[-1] // self.head_dim, k.shape[-1] // self.head_dim
        q, k, v = q.view(b, s, hq, self.head_dim), k.view(b, s, hkv, self.head_dim), v.view(b, s, hkv, self.head_dim)
        from oslo_b200.ops.attention import decode_offset

        off = decode_offset()
        cos, sin = self._tables(s + off, x.device)
        pos = (torch.arange(s, device=x.device) + off).repeat(b) if off else None  # incremental decoding
        q = OF.apply_rope(q, cos, sin, self.head_dim, neox=True, positions=pos)
        k = OF.apply_rope(k, cos, sin, self.head_dim, neox=True, positions=pos)
        if hkv != hq:
            rep = hq // hkv
            k = k.repeat_interleave(rep, dim=2)
            v = v.repeat_interleave(rep, dim=2)
        ctx = OF.attention(q, k, v, causal=True, mask=attention_mask)
        return self.o_proj(ctx)


class LlamaMLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.gate_proj = onn.Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.up_proj = onn.Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.down_proj = onn.Linear(config.intermediate_size, config.hidden_size, bias=False)

    def forward(self, x):
        return self.down_proj(swiglu2(self.gate_proj(x), self.up_proj(x)))


class LlamaDecoderLayer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.self_attn = LlamaAttention(config)
        self.mlp = LlamaMLP(config)
        self.input_layernorm = onn.FusedRMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = onn.FusedRMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, x, attention_mask=None):
        x = x + self.self_attn(self.input_layernorm(x), attention_mask)
        return x + self.mlp(self.post_attention_layernorm(x))


class LlamaModel(PreTrainedModel):
    config_class = LlamaConfig

    def __init__(self, config):
        super().__init__(config)
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([LlamaDecoderLayer(config) for _ in range(config.num_hidden_layers)])
        self.norm = onn.FusedRMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.gradient_checkpointing = False

    def get_input_embeddings(self):
        return self.embed_tokens

    def forward(self, input_ids, attention_mask=None):
        x = self.embed_tokens(input_ids)
        for layer in self.layers:
            if self.gradient_checkpointing and self.training:
                x = torch.utils.checkpoint.checkpoint(layer, x, attention_mask, use_reentrant=False)
            else:
                x = layer(x, attention_mask)
        return self.norm(x)


class LlamaForCausalLM(PreTrainedModel):
    config_class = LlamaConfig
    base_model_prefix = "model"

    def __init__(self, config):
        super().__init__(config)
        self.model = LlamaModel(config)
        self.lm_head = onn.Linear(config.hidden_size, config.vocab_size, bias=False)
        self.post_init()

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def get_output_embeddings(self):
        return self.lm_head

    def gradient_checkpointing_enable(self):
        self.model.gradient_checkpointing = True

    def pipeline_units(self):
        from oslo_b200.parallel.pipeline_parallel.partitioner import PipeUnit

        base = self.model

        def embed(state):
            state["hidden"] = base.embed_tokens(state["input_ids"])
            return state

        def make_layer(layer):
            def run(state):
                state["hidden"] = layer(state["hidden"], state.get("attention_mask"))
                return state

            return run

        def head(state):
            logits = self.lm_head(base.norm(state["hidden"]))
            state["logits"] = logits
            if state.get("labels") is not None:
                from .losses import causal_lm_loss

                res = causal_lm_loss(self, logits, state["labels"])
                state["loss"] = res.value
                if res.consumed_logits:
                    state["logits"] = None
            return state

        units = [PipeUnit("embed_tokens", [base.embed_tokens], embed)]
        units += [PipeUnit(f"layers.{i}", [l], make_layer(l)) for i, l in enumerate(base.layers)]
        units.append(PipeUnit("head", [base.norm, self.lm_head], head))
        return units

    def forward(self, input_ids=None, attention_mask=None, labels=None, **kwargs):
        hidden = self.model(input_ids, attention_mask)
        chunk = getattr(self.config, "chunked_head_loss", 0)
        if labels is not None and chunk:  # config.chunked_head_loss = tokens per chunk: the logits are never materialised
            from .losses import chunked_head_loss

            loss = chunked_head_loss(self, hidden, self.lm_head, labels, chunk)
            if loss is not None:
                return CausalLMOutput(loss=loss, logits=None)
        logits = self.lm_head(hidden)
        loss = None
        if labels is not None:
            from .losses import causal_lm_loss

            res = causal_lm_loss(self, logits, labels)
            loss, logits = res.value, (None if res.consumed_logits else logits)
        return CausalLMOutput(loss=loss, logits=logits)
