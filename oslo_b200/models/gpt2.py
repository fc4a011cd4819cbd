"""GPT-2 style decoder (learned positions, LayerNorm, fused ``c_attn`` in ``[in, 3*out]`` Conv1D layout, GELU MLP).

State-dict names and weight layouts follow Hugging Face ``GPT2LMHeadModel`` (``transformer.h.N.attn.c_attn.weight``
is ``[n_embd, 3 n_embd]``; ``lm_head.weight`` is tied to ``transformer.wte.weight``), so its checkpoints load directly.
Parity: the reference's patched copy, oslo/transformers/models/gpt2/modeling_gpt2.py:81-88,309-323,725-880.
"""
from __future__ import annotations

import torch
import torch.nn as nn

import oslo_b200.nn as onn
from oslo_b200.nn import functional as OF

from .config import GPT2Config
from .modeling_utils import CausalLMOutput, PreTrainedModel


class GPT2Attention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.embed_dim = config.n_embd
        self.num_heads = config.n_head
        self.head_dim = config.n_embd // config.n_head
        self.c_attn = onn.Conv1D(3 * config.n_embd, config.n_embd)
        self.c_proj = onn.Conv1D(config.n_embd, config.n_embd, skip_bias_add=True)

    def forward(self, hidden_states, attention_mask=None):
        qkv = self.c_attn(hidden_states)  # [b, s, 3 * heads_local * hd], laid out [3, heads, hd]
        heads = qkv.shape[-1] // (3 * self.head_dim)
        ctx = OF.qkv_attention(qkv, heads, self.head_dim, layout="3hd", causal=True, mask=attention_mask)
        return self.c_proj(ctx)


class GPT2MLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        inner = config.n_inner or 4 * config.n_embd
        self.c_fc = onn.Conv1D(inner, config.n_embd, skip_bias_add=True)
        self.c_proj = onn.Conv1D(config.n_embd, inner, skip_bias_add=True)

    def forward(self, hidden_states):
        h, bias = self.c_fc(hidden_states)
        h = OF.bias_gelu(h, bias)
        return self.c_proj(h)


class GPT2Block(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.ln_1 = onn.FusedLayerNorm(config.n_embd, eps=config.layer_norm_epsilon)
        self.attn = GPT2Attention(config)
        self.ln_2 = onn.FusedLayerNorm(config.n_embd, eps=config.layer_norm_epsilon)
        self.mlp = GPT2MLP(config)
        self.resid_pdrop = config.resid_pdrop

    def forward(self, x, attention_mask=None):
        a, a_bias = self.attn(self.ln_1(x), attention_mask)
        x = OF.bias_dropout_add(a, a_bias, x, self.resid_pdrop, self.training)
        m, m_bias = self.mlp(self.ln_2(x))
        return OF.bias_dropout_add(m, m_bias, x, self.resid_pdrop, self.training)


class GPT2Model(PreTrainedModel):
    config_class = GPT2Config

    def __init__(self, config):
        super().__init__(config)
        self.wte = nn.Embedding(config.vocab_size, config.n_embd)
        self.wpe = nn.Embedding(config.n_positions, config.n_embd)
        self.drop = nn.Dropout(config.embd_pdrop)
        self.h = nn.ModuleList([GPT2Block(config) for _ in range(config.n_layer)])
        self.ln_f = onn.FusedLayerNorm(config.n_embd, eps=config.layer_norm_epsilon)
        self.gradient_checkpointing = False

    def get_input_embeddings(self):
        return self.wte

    def forward(self, input_ids, attention_mask=None, position_ids=None):
        s = input_ids.shape[-1]
        if position_ids is None:
            from oslo_b200.ops.attention import decode_offset

            position_ids = (torch.arange(s, device=input_ids.device) + decode_offset()).unsqueeze(0)
        x = self.wte(input_ids)
        pos = self.wpe(position_ids)
        if pos.shape[:-1] != x.shape[:-1] and pos.shape[0] != 1:
            from .gpt_neox import _sp_like

            pos = _sp_like(pos, x, self)
        elif pos.shape[-1] != x.shape[-1] or (pos.shape[0] == 1 and pos.shape[1] != x.shape[1]):
            from .gpt_neox import _sp_like

            pos = _sp_like(pos.expand(input_ids.shape[0], -1, -1), x, self)
        x = self.drop(x + pos)
        for block in self.h:
            if self.gradient_checkpointing and self.training:
                x = torch.utils.checkpoint.checkpoint(block, x, attention_mask, use_reentrant=False)
            else:
                x = block(x, attention_mask)
        return self.ln_f(x)


class GPT2LMHeadModel(PreTrainedModel):
    config_class = GPT2Config
    base_model_prefix = "transformer"

    def __init__(self, config):
        super().__init__(config)
        self.transformer = GPT2Model(config)
        self.lm_head = onn.Linear(config.n_embd, config.vocab_size, bias=False)
        self.post_init()

    def get_input_embeddings(self):
        return self.transformer.wte

    def get_output_embeddings(self):
        return self.lm_head

    def gradient_checkpointing_enable(self):
        self.transformer.gradient_checkpointing = True

    def pipeline_units(self):
        from oslo_b200.parallel.pipeline_parallel.partitioner import PipeUnit

        base = self.transformer

        def embed(state):
            ids = state["input_ids"]
            pos = torch.arange(ids.shape[-1], device=ids.device).unsqueeze(0)
            state["hidden"] = base.drop(base.wte(ids) + base.wpe(pos))
            return state

        def make_layer(block):
            def run(state):
                state["hidden"] = block(state["hidden"], state.get("attention_mask"))
                return state

            return run

        def head(state):
            logits = self.lm_head(base.ln_f(state["hidden"]))
            state["logits"] = logits
            if state.get("labels") is not None:
                from .losses import causal_lm_loss

                res = causal_lm_loss(self, logits, state["labels"])
                state["loss"] = res.value
                if res.consumed_logits:
                    state["logits"] = None
            return state

        units = [PipeUnit("embed", [base.wte, base.wpe], embed)]
        units += [PipeUnit(f"h.{i}", [b], make_layer(b)) for i, b in enumerate(base.h)]
        units.append(PipeUnit("head", [base.ln_f, self.lm_head], head))
        return units

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, labels=None, **kwargs):
        hidden = self.transformer(input_ids, attention_mask, position_ids)
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


class MoEGPTLMHeadModel(GPT2LMHeadModel):
    """GPT-2 style decoder intended for :class:`oslo_b200.parallel.ExpertParallel`, which turns the FFN of the layers
    chosen by ``config.moe_every`` into mixtures of ``config.num_experts`` experts."""

    def moe_layer_ids(self):
        every = getattr(self.config, "moe_every", 2)
        return [i for i in range(self.config.n_layer) if i % every == every - 1]
