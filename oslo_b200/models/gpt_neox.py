"""GPT-NeoX style decoder (rotary on a fraction of the head dim, parallel attention + MLP residual).

State-dict names follow Hugging Face ``GPTNeoXForCausalLM`` (``gpt_neox.layers.N.attention.query_key_value`` ...,
``embed_out``); the fused QKV projection is laid out ``[heads, 3, head_dim]`` as there.  The model is written
against :mod:`oslo_b200.nn` so every GEMM / norm / activation / softmax runs the sm_100a kernels on CUDA, and
so the tensor-parallel wrapper can swap its linears for sharded ones by name.
"""
from __future__ import annotations

import torch
import torch.nn as nn

import oslo_b200.nn as onn
from oslo_b200.nn import functional as OF

from .config import GPTNeoXConfig
from .modeling_utils import CausalLMOutput, PreTrainedModel


def _sp_like(t, ref, module):
    """Shard ``t`` (full batch) like ``ref`` when the model runs token-sharded between its linears."""
    sp = getattr(module, "sequence_parallel_state", None)
    if sp is None or t.shape[: ref.dim() - 1] == ref.shape[:-1]:
        return t
    return sp.shard(t)


class GPTNeoXAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.num_attention_heads = config.num_attention_heads
        self.hidden_size = config.hidden_size
        self.head_size = config.hidden_size // config.num_attention_heads
        self.rotary_ndims = int(self.head_size * config.rotary_pct)
        self.rotary_base = config.rotary_emb_base
        self.max_positions = config.max_position_embeddings
        self.query_key_value = onn.Linear(config.hidden_size, 3 * config.hidden_size)
        self.dense = onn.Linear(config.hidden_size, config.hidden_size, skip_bias_add=True)
        self._rope = None

    def _tables(self, seq, device):
        if self._rope is None or self._rope[0].shape[0] < seq or self._rope[0].device != device:
            n = max(seq, self.max_positions)
            self._rope = OF.rope_tables(n, self.rotary_ndims, self.rotary_base, device)
        # rows [0, seq): the kernels take a token's position as (flattened token index) mod (table rows)
        return self._rope[0][:seq], self._rope[1][:seq]

    def forward(self, hidden_states, attention_mask=None):
        qkv = self.query_key_value(hidden_states)  # [b, s, heads_local * 3 * hd]
        return self.dense(self.core(qkv, attention_mask))  # (out, bias)

    def core(self, qkv, attention_mask=None):
        """Rotary embedding + causal attention on an already projected ``[b, s, heads_local * 3 * hd]`` tensor."""
        b, s = qkv.shape[0], qkv.shape[1]
        heads = qkv.shape[-1] // (3 * self.head_size)
        rope = None
        if self.rotary_ndims > 0:
            from oslo_b200.ops.attention import decode_offset

            cos, sin = self._tables(s + decode_offset(), qkv.device)  # incremental decoding rotates at offset positions
            rope = (cos, sin, self.rotary_ndims, True)
        return OF.qkv_attention(qkv, heads, self.head_size, layout="h3d", causal=True, rope=rope, mask=attention_mask)


#: apply gelu'(pre-activation) in the epilogue of the gradient GEMM of the sequence-parallel paired block instead of in a
#: pass of its own.  Off by default: on two B200s the 1.3B step took 88.7 / 89.4 ms without it and 90.6 / 91.4 ms with it
#: (the epilogue's extra 16-byte aux reads stretch the fused all-gather GEMM more than the separate pass costs).
#: OSLO_B200_DEFER_GELU=1 switches it on.
_DEFER_GELU_GRAD = __import__("os").environ.get("OSLO_B200_DEFER_GELU", "0") == "1"


class GPTNeoXMLP(nn.Module):
    #: the forward hands its linears' weights to one fused op instead of calling the linears: engines that materialise
    #: parameters per module call (chunked ZeRO-3) must treat this module's whole subtree as one unit
    reads_descendant_parameters = True

    def __init__(self, config):
        super().__init__()
        self.dense_h_to_4h = onn.Linear(config.hidden_size, config.intermediate_size, skip_bias_add=True)
        self.dense_4h_to_h = onn.Linear(config.intermediate_size, config.hidden_size, skip_bias_add=True)

    def forward(self, hidden_states):
        up, down = self.dense_h_to_4h, self.dense_4h_to_h
        if type(up) is onn.Linear and type(down) is onn.Linear and not up.reversed and not down.reversed and down.skip_bias_add:
            from oslo_b200.ops.gemm import mlp_gelu

            # both element-wise steps ride in GEMM epilogues: bias + GELU forward, GELU' in the gradient GEMM backward
            return mlp_gelu(hidden_states, up.weight, up.bias, down.weight), down.bias
        if type(up) is onn.Linear and not up.reversed:
            from oslo_b200.ops.gemm import linear_gelu

            h = linear_gelu(hidden_states, up.weight, up.bias)  # bias + GELU in the GEMM epilogue
        else:
            h, bias = up(hidden_states)
            h = OF.bias_gelu(h, bias)
        return self.dense_4h_to_h(h)  # (out, bias)


class GPTNeoXLayer(nn.Module):
    reads_descendant_parameters = True  # the paired (parallel-residual) path reads attention and MLP weights directly

    def __init__(self, config):
        super().__init__()
        self.use_parallel_residual = config.use_parallel_residual
        self.input_layernorm = onn.FusedLayerNorm(config.hidden_size, eps=config.layer_norm_eps)
        self.post_attention_layernorm = onn.FusedLayerNorm(config.hidden_size, eps=config.layer_norm_eps)
        self.attention = GPTNeoXAttention(config)
        self.mlp = GPTNeoXMLP(config)
        self.hidden_dropout = config.hidden_dropout

    def _paired_ok(self) -> bool:
        """Sequence-parallel 1-D layers with a parallel residual and no active dropout: the two column linears share
        one all-gather and the two row linears one reduce-scatter."""
        qkv = self.attention.query_key_value
        return (self.use_parallel_residual and getattr(qkv, "sequence_parallel", False)
                and getattr(qkv, "world_size", 1) > 1 and not (self.training and self.hidden_dropout > 0)
                and getattr(self.mlp.dense_4h_to_h, "sequence_parallel", False)
                and self.input_layernorm.elementwise_affine and not qkv.reversed)

    def _forward_paired(self, x, attention_mask):
        """Parallel-residual block with HALF the NVLink traffic of four independent sequence-parallel linears.

        Both LayerNorms normalise the same ``x``; they differ only in their affine parameters, which are folded into
        the weights that consume them (``W (g * xhat + b) = (W diag(g)) xhat + W b``).  So the normalised shard
        ``xhat`` is all-gathered ONCE and feeds both column linears, and the attention and MLP row products are summed
        locally before ONE reduce-scatter.  Backward mirrors this: one all-gather of ``dY`` serves both row linears
        and ``d xhat`` of both column linears leaves in one reduce-scatter.  The folds are ordinary autograd ops on
        the (small, sharded) weights, so gradients of the LayerNorm parameters need no special handling."""
        from oslo_b200.ops.norm import layer_norm
        from oslo_b200.parallel.tensor_parallel import _ops_1d as ops

        att, mlp = self.attention, self.mlp
        ln1, ln2 = self.input_layernorm, self.post_attention_layernorm
        qkv_l, h4h = att.query_key_value, mlp.dense_h_to_4h
        pc, tp = qkv_l.parallel_context, qkv_l.world_size
        lead = list(x.shape[:-1])
        hidden = x.shape[-1]
        xhat = layer_norm(x, (hidden,), None, None, ln1.eps).reshape(-1, hidden)
        w1 = qkv_l.weight * ln1.weight.to(qkv_l.weight.dtype)
        b1 = torch.mv(qkv_l.weight, ln1.bias.to(qkv_l.weight.dtype))
        if qkv_l.bias is not None:
            b1 = b1 + qkv_l.bias
        w2 = h4h.weight * ln2.weight.to(h4h.weight.dtype)
        b2 = torch.mv(h4h.weight, ln2.bias.to(h4h.weight.dtype))
        if h4h.bias is not None:
            b2 = b2 + h4h.bias
        if _DEFER_GELU_GRAD:
            qkv, h, h_pre = ops.ag_linear_pair(xhat, w1, w2, pc, b1, b2, gelu2="deferred")
        else:
            (qkv, h), h_pre = ops.ag_linear_pair(xhat, w1, w2, pc, b1, b2, gelu2=True), None
        d = att.query_key_value.sequence_parallel_state.dim if getattr(att.query_key_value, "sequence_parallel_state", None) else 0
        full = list(lead)
        full[d] *= tp
        qkv = qkv.view(*full, qkv.shape[-1])
        ctx = att.core(qkv, attention_mask)
        out = ops.linear_pair_rs(ctx.reshape(-1, ctx.shape[-1]), att.dense.weight, h, mlp.dense_4h_to_h.weight, pc, x2_pre=h_pre)
        out = out.view(*lead, hidden)
        bias = None
        for b in (att.dense.bias, mlp.dense_4h_to_h.bias):
            if b is not None:
                bias = b if bias is None else bias + b
        return OF.bias_dropout_add(out, bias, x, 0.0, False)

    def forward(self, hidden_states, attention_mask=None):
        if self._paired_ok():
            return self._forward_paired(hidden_states, attention_mask)
        attn, attn_bias = self.attention(self.input_layernorm(hidden_states), attention_mask)
        p, tr = self.hidden_dropout, self.training
        if self.use_parallel_residual:
            mlp, mlp_bias = self.mlp(self.post_attention_layernorm(hidden_states))
            x = OF.bias_dropout_add(attn, attn_bias, hidden_states, p, tr)
            return OF.bias_dropout_add(mlp, mlp_bias, x, p, tr)
        x = OF.bias_dropout_add(attn, attn_bias, hidden_states, p, tr)
        mlp, mlp_bias = self.mlp(self.post_attention_layernorm(x))
        return OF.bias_dropout_add(mlp, mlp_bias, x, p, tr)


class GPTNeoXModel(PreTrainedModel):
    config_class = GPTNeoXConfig

    def __init__(self, config):
        super().__init__(config)
        self.embed_in = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([GPTNeoXLayer(config) for _ in range(config.num_hidden_layers)])
        self.final_layer_norm = onn.FusedLayerNorm(config.hidden_size, eps=config.layer_norm_eps)
        self.gradient_checkpointing = False

    def get_input_embeddings(self):
        return self.embed_in

    def forward(self, input_ids, attention_mask=None):
        x = self.embed_in(input_ids)
        for layer in self.layers:
            if self.gradient_checkpointing and self.training:
                x = torch.utils.checkpoint.checkpoint(layer, x, attention_mask, use_reentrant=False)
            else:
                x = layer(x, attention_mask)
        return self.final_layer_norm(x)


class GPTNeoXForCausalLM(PreTrainedModel):
    config_class = GPTNeoXConfig
    base_model_prefix = "gpt_neox"

    def __init__(self, config):
        super().__init__(config)
        self.gpt_neox = GPTNeoXModel(config)
        self.embed_out = onn.Linear(config.hidden_size, config.vocab_size, bias=False)
        self.post_init()

    def get_input_embeddings(self):
        return self.gpt_neox.embed_in

    def get_output_embeddings(self):
        return self.embed_out

    def gradient_checkpointing_enable(self):
        self.gpt_neox.gradient_checkpointing = True

    def pipeline_units(self):
        """Embedding, one unit per layer, then final norm + head + loss."""
        from oslo_b200.parallel.pipeline_parallel.partitioner import PipeUnit

        base = self.gpt_neox

        def embed(state):
            state["hidden"] = base.embed_in(state["input_ids"])
            return state

        def make_layer(layer):
            def run(state):
                state["hidden"] = layer(state["hidden"], state.get("attention_mask"))
                return state

            return run

        def head(state):
            logits = self.embed_out(base.final_layer_norm(state["hidden"]))
            state["logits"] = logits
            if state.get("labels") is not None:
                from .losses import causal_lm_loss

                res = causal_lm_loss(self, logits, state["labels"])
                state["loss"] = res.value
                if res.consumed_logits:
                    state["logits"] = None
            return state

        units = [PipeUnit("embed_in", [base.embed_in], embed)]
        units += [PipeUnit(f"layers.{i}", [l], make_layer(l)) for i, l in enumerate(base.layers)]
        units.append(PipeUnit("head", [base.final_layer_norm, self.embed_out], head))
        return units

    def forward(self, input_ids=None, attention_mask=None, labels=None, **kwargs):
        hidden = self.gpt_neox(input_ids, attention_mask)
        chunk = getattr(self.config, "chunked_head_loss", 0)
        if labels is not None and chunk:  # config.chunked_head_loss = tokens per chunk: the logits are never materialised
            from .losses import chunked_head_loss

            loss = chunked_head_loss(self, hidden, self.embed_out, labels, chunk)
            if loss is not None:
                return CausalLMOutput(loss=loss, logits=None)
        logits = self.embed_out(hidden)
        loss = None
        if labels is not None:
            from .losses import causal_lm_loss

            loss = causal_lm_loss(self, logits, labels)
            logits = None if loss.consumed_logits else logits
            loss = loss.value
        return CausalLMOutput(loss=loss, logits=logits)
