"""DistilBERT: a post-LayerNorm encoder without token types or pooler.

Names follow Hugging Face ``DistilBert*`` (``distilbert.transformer.layer.N.attention.q_lin`` ...), so its checkpoints
and the built-in tensor-parallel table (``q_lin / k_lin / v_lin / lin1`` column, ``out_lin / lin2`` row,
``n_heads`` / ``dim`` divided) apply.  Parity: oslo/transformers/models/distilbert/modeling_distilbert.py.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

import oslo_b200.nn as onn
from oslo_b200.nn import functional as OF

from .config import DistilBertConfig
from .heads import classification_loss, qa_loss
from .losses import token_lm_loss
from .modeling_utils import ModelOutput, PreTrainedModel, additive_mask


class Embeddings(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.word_embeddings = nn.Embedding(config.vocab_size, config.dim, padding_idx=config.pad_token_id)
        self.position_embeddings = nn.Embedding(config.max_position_embeddings, config.dim)
        self.LayerNorm = onn.FusedLayerNorm(config.dim, eps=1e-12)
        self.dropout = nn.Dropout(config.dropout)

    def forward(self, input_ids):
        pos = torch.arange(input_ids.shape[1], device=input_ids.device).unsqueeze(0)
        return self.dropout(self.LayerNorm(self.word_embeddings(input_ids) + self.position_embeddings(pos)))


class MultiHeadSelfAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.n_heads, self.dim = config.n_heads, config.dim
        self.head_dim = config.dim // config.n_heads
        self.q_lin = onn.Linear(config.dim, config.dim)
        self.k_lin = onn.Linear(config.dim, config.dim)
        self.v_lin = onn.Linear(config.dim, config.dim)
        self.out_lin = onn.Linear(config.dim, config.dim, skip_bias_add=True)

    def forward(self, x, mask=None):
        b, s, _ = x.shape
        q, k, v = (lin(x).unflatten(-1, (-1, self.head_dim)) for lin in (self.q_lin, self.k_lin, self.v_lin))
        return self.out_lin(OF.attention(q, k, v, causal=False, mask=mask))


class FFN(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.lin1 = onn.Linear(config.dim, config.hidden_dim, skip_bias_add=True)
        self.lin2 = onn.Linear(config.hidden_dim, config.dim, skip_bias_add=True)
        self.act = config.activation

    def forward(self, x):
        h, bias = self.lin1(x)
        return self.lin2(OF.bias_act(h, bias, self.act))


class TransformerBlock(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.attention = MultiHeadSelfAttention(config)
        self.sa_layer_norm = onn.FusedLayerNorm(config.dim, eps=1e-12)
        self.ffn = FFN(config)
        self.output_layer_norm = onn.FusedLayerNorm(config.dim, eps=1e-12)
        self.p = config.dropout

    def forward(self, x, mask=None):
        a, a_bias = self.attention(x, mask)
        x = self.sa_layer_norm(OF.bias_dropout_add(a, a_bias, x, 0.0, self.training))
        f, f_bias = self.ffn(x)
        return self.output_layer_norm(OF.bias_dropout_add(f, f_bias, x, self.p, self.training))


class Transformer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.layer = nn.ModuleList([TransformerBlock(config) for _ in range(config.n_layers)])
        self.gradient_checkpointing = False

    def forward(self, x, mask=None):
        for layer in self.layer:
            if self.gradient_checkpointing and self.training:
                x = torch.utils.checkpoint.checkpoint(layer, x, mask, use_reentrant=False)
            else:
                x = layer(x, mask)
        return x


class DistilBertPreTrainedModel(PreTrainedModel):
    config_class = DistilBertConfig
    base_model_prefix = "distilbert"

    def get_input_embeddings(self):
        return getattr(self, "distilbert", self).embeddings.word_embeddings

    def gradient_checkpointing_enable(self):
        getattr(self, "distilbert", self).transformer.gradient_checkpointing = True


class DistilBertModel(DistilBertPreTrainedModel):
    def __init__(self, config):
        super().__init__(config)
        self.embeddings = Embeddings(config)
        self.transformer = Transformer(config)
        self.post_init()

    def forward(self, input_ids, attention_mask=None, **unused):
        x = self.transformer(self.embeddings(input_ids), additive_mask(attention_mask, torch.float32))
        return ModelOutput(last_hidden_state=x)


class DistilBertForMaskedLM(DistilBertPreTrainedModel):
    def __init__(self, config):
        super().__init__(config)
        self.distilbert = DistilBertModel(config)
        self.vocab_transform = onn.Linear(config.dim, config.dim, skip_bias_add=True)
        self.vocab_layer_norm = onn.FusedLayerNorm(config.dim, eps=1e-12)
        self.vocab_projector = onn.Linear(config.dim, config.vocab_size)
        self.post_init()

    def get_output_embeddings(self):
        return self.vocab_projector

    def forward(self, input_ids, attention_mask=None, labels=None, **unused):
        x = self.distilbert(input_ids, attention_mask).last_hidden_state
        h, bias = self.vocab_transform(x)
        logits = self.vocab_projector(self.vocab_layer_norm(OF.bias_act(h, bias, self.config.activation)))
        loss = None
        if labels is not None:
            res = token_lm_loss(self, logits, labels)
            loss, logits = res.value, (None if res.consumed_logits else logits)
        return ModelOutput(loss=loss, logits=logits)


class DistilBertForSequenceClassification(DistilBertPreTrainedModel):
    def __init__(self, config):
        super().__init__(config)
        self.num_labels = config.num_labels
        self.distilbert = DistilBertModel(config)
        self.pre_classifier = onn.Linear(config.dim, config.dim)
        self.classifier = onn.Linear(config.dim, config.num_labels)
        self.dropout = nn.Dropout(config.seq_classif_dropout)
        self.post_init()

    def forward(self, input_ids, attention_mask=None, labels=None, **unused):
        x = self.distilbert(input_ids, attention_mask).last_hidden_state[:, 0]
        logits = self.classifier(self.dropout(F.relu(self.pre_classifier(x))))
        return ModelOutput(loss=classification_loss(logits, labels, self.num_labels), logits=logits)


class DistilBertForTokenClassification(DistilBertPreTrainedModel):
    def __init__(self, config):
        super().__init__(config)
        self.num_labels = config.num_labels
        self.distilbert = DistilBertModel(config)
        self.dropout = nn.Dropout(config.dropout)
        self.classifier = onn.Linear(config.dim, config.num_labels)
        self.post_init()

    def forward(self, input_ids, attention_mask=None, labels=None, **unused):
        logits = self.classifier(self.dropout(self.distilbert(input_ids, attention_mask).last_hidden_state))
        loss = None
        if labels is not None:
            loss = F.cross_entropy(logits.reshape(-1, self.num_labels).float(), labels.reshape(-1), ignore_index=-100)
        return ModelOutput(loss=loss, logits=logits)


class DistilBertForQuestionAnswering(DistilBertPreTrainedModel):
    def __init__(self, config):
        super().__init__(config)
        self.distilbert = DistilBertModel(config)
        self.qa_outputs = onn.Linear(config.dim, 2)
        self.dropout = nn.Dropout(config.qa_dropout)
        self.post_init()

    def forward(self, input_ids, attention_mask=None, start_positions=None, end_positions=None, **unused):
        x = self.dropout(self.distilbert(input_ids, attention_mask).last_hidden_state)
        start, end = (t.squeeze(-1).contiguous() for t in self.qa_outputs(x).split(1, dim=-1))
        return ModelOutput(loss=qa_loss(start, end, start_positions, end_positions), start_logits=start, end_logits=end)


class DistilBertForMultipleChoice(DistilBertPreTrainedModel):
    def __init__(self, config):
        super().__init__(config)
        self.distilbert = DistilBertModel(config)
        self.pre_classifier = onn.Linear(config.dim, config.dim)
        self.classifier = onn.Linear(config.dim, 1)
        self.dropout = nn.Dropout(config.seq_classif_dropout)
        self.post_init()

    def forward(self, input_ids, attention_mask=None, labels=None, **unused):
        n = input_ids.shape[1]
        flat = lambda t: t.reshape(-1, t.shape[-1]) if t is not None else None  # noqa: E731
        x = self.distilbert(flat(input_ids), flat(attention_mask)).last_hidden_state[:, 0]
        logits = self.classifier(self.dropout(F.relu(self.pre_classifier(x)))).view(-1, n)
        loss = F.cross_entropy(logits.float(), labels) if labels is not None else None
        return ModelOutput(loss=loss, logits=logits)


__all__ = [n for n in globals() if n.startswith("DistilBert") and not n.endswith("Config")]
