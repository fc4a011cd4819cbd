"""ALBERT: factorised embeddings and one (or a few) layer groups whose weights are reused at every depth.

Names follow Hugging Face ``Albert*`` (``albert.encoder.albert_layer_groups.G.albert_layers.I.attention.query`` ...).
Parity: oslo/transformers/models/albert/modeling_albert.py.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

import oslo_b200.nn as onn
from oslo_b200.nn import functional as OF

from .bert import BertEmbeddings, make_task_models
from .config import AlbertConfig
from .losses import token_lm_loss
from .modeling_utils import ModelOutput, PreTrainedModel, additive_mask


class AlbertAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.num_attention_heads = config.num_attention_heads
        self.attention_head_size = config.hidden_size // config.num_attention_heads
        self.all_head_size = config.hidden_size
        self.query = onn.Linear(config.hidden_size, config.hidden_size)
        self.key = onn.Linear(config.hidden_size, config.hidden_size)
        self.value = onn.Linear(config.hidden_size, config.hidden_size)
        self.dense = onn.Linear(config.hidden_size, config.hidden_size, skip_bias_add=True)
        self.LayerNorm = onn.FusedLayerNorm(config.hidden_size, eps=config.layer_norm_eps)
        self.p = config.hidden_dropout_prob

    def forward(self, x, mask=None):
        b, s, _ = x.shape
        q, k, v = (lin(x).unflatten(-1, (-1, self.attention_head_size)) for lin in (self.query, self.key, self.value))
        h, bias = self.dense(OF.attention(q, k, v, causal=False, mask=mask))
        return self.LayerNorm(OF.bias_dropout_add(h, bias, x, self.p, self.training))


class AlbertLayer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.attention = AlbertAttention(config)
        self.ffn = onn.Linear(config.hidden_size, config.intermediate_size, skip_bias_add=True)
        self.ffn_output = onn.Linear(config.intermediate_size, config.hidden_size, skip_bias_add=True)
        self.full_layer_layer_norm = onn.FusedLayerNorm(config.hidden_size, eps=config.layer_norm_eps)
        self.act, self.p = config.hidden_act, config.hidden_dropout_prob

    def forward(self, x, mask=None):
        a = self.attention(x, mask)
        h, bias = self.ffn(a)
        o, o_bias = self.ffn_output(OF.bias_act(h, bias, self.act))
        return self.full_layer_layer_norm(OF.bias_dropout_add(o, o_bias, a, self.p, self.training))


class AlbertLayerGroup(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.albert_layers = nn.ModuleList([AlbertLayer(config) for _ in range(config.inner_group_num)])

    def forward(self, x, mask=None):
        for layer in self.albert_layers:
            x = layer(x, mask)
        return x


class AlbertTransformer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.embedding_hidden_mapping_in = onn.Linear(config.embedding_size, config.hidden_size)
        self.albert_layer_groups = nn.ModuleList([AlbertLayerGroup(config) for _ in range(config.num_hidden_groups)])
        self.gradient_checkpointing = False

    def forward(self, x, mask=None):
        x = self.embedding_hidden_mapping_in(x)
        n, g = self.config.num_hidden_layers, self.config.num_hidden_groups
        for i in range(n):
            group = self.albert_layer_groups[int(i / (n / g))]
            if self.gradient_checkpointing and self.training:
                x = torch.utils.checkpoint.checkpoint(group, x, mask, use_reentrant=False)
            else:
                x = group(x, mask)
        return x


class AlbertPreTrainedModel(PreTrainedModel):
    config_class = AlbertConfig
    base_model_prefix = "albert"

    def get_input_embeddings(self):
        return getattr(self, "albert", self).embeddings.word_embeddings

    def gradient_checkpointing_enable(self):
        getattr(self, "albert", self).encoder.gradient_checkpointing = True


class AlbertModel(AlbertPreTrainedModel):
    def __init__(self, config, add_pooling_layer=True):
        super().__init__(config)
        self.embeddings = BertEmbeddings(config, embedding_size=config.embedding_size)
        self.encoder = AlbertTransformer(config)
        self.pooler = onn.Linear(config.hidden_size, config.hidden_size) if add_pooling_layer else None
        self.post_init()

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, position_ids=None, **unused):
        x = self.encoder(self.embeddings(input_ids, token_type_ids, position_ids), additive_mask(attention_mask, torch.float32))
        pooled = torch.tanh(self.pooler(x[:, 0])) if self.pooler is not None else None
        return ModelOutput(last_hidden_state=x, pooler_output=pooled)


class AlbertMLMHead(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.LayerNorm = onn.FusedLayerNorm(config.embedding_size, eps=config.layer_norm_eps)
        self.dense = onn.Linear(config.hidden_size, config.embedding_size, skip_bias_add=True)
        self.decoder = onn.Linear(config.embedding_size, config.vocab_size)
        self.bias = self.decoder.bias
        self.act = config.hidden_act

    def forward(self, x):
        h, bias = self.dense(x)
        return self.decoder(self.LayerNorm(OF.bias_act(h, bias, self.act)))


class AlbertForMaskedLM(AlbertPreTrainedModel):
    def __init__(self, config):
        super().__init__(config)
        self.albert = AlbertModel(config, add_pooling_layer=False)
        self.predictions = AlbertMLMHead(config)
        self.post_init()

    def get_output_embeddings(self):
        return self.predictions.decoder

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, position_ids=None, labels=None, **unused):
        x = self.albert(input_ids, attention_mask, token_type_ids, position_ids).last_hidden_state
        logits = self.predictions(x)
        loss = None
        if labels is not None:
            res = token_lm_loss(self, logits, labels)
            loss, logits = res.value, (None if res.consumed_logits else logits)
        return ModelOutput(loss=loss, logits=logits)


class AlbertSOPHead(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dropout = nn.Dropout(config.classifier_dropout_prob)
        self.classifier = onn.Linear(config.hidden_size, config.num_labels)

    def forward(self, pooled):
        return self.classifier(self.dropout(pooled))


class AlbertForPreTraining(AlbertPreTrainedModel):
    """Masked-LM plus sentence-order prediction."""

    def __init__(self, config):
        super().__init__(config)
        self.albert = AlbertModel(config)
        self.predictions = AlbertMLMHead(config)
        self.sop_classifier = AlbertSOPHead(config)
        self.post_init()

    def get_output_embeddings(self):
        return self.predictions.decoder

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, position_ids=None, labels=None,
                sentence_order_label=None, **unused):
        out = self.albert(input_ids, attention_mask, token_type_ids, position_ids)
        logits, sop = self.predictions(out.last_hidden_state), self.sop_classifier(out.pooler_output)
        loss = None
        if labels is not None and sentence_order_label is not None:
            loss = F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), labels.reshape(-1), ignore_index=-100) \
                + F.cross_entropy(sop.float(), sentence_order_label.view(-1))
        return ModelOutput(loss=loss, prediction_logits=logits, sop_logits=sop)


def _task_config(config):
    """The shared task heads read ``classifier_dropout``; ALBERT's configuration calls it ``classifier_dropout_prob``."""
    if getattr(config, "classifier_dropout", None) is None:
        config.classifier_dropout = config.classifier_dropout_prob
    return config


_tasks = make_task_models("Albert", AlbertModel, AlbertPreTrainedModel, module=__name__)
for _name, _cls in _tasks.items():
    _orig = _cls.__init__

    def _init(self, config, _orig=_orig):
        _orig(self, _task_config(config))

    _cls.__init__ = _init
globals().update(_tasks)

__all__ = [n for n in globals() if n.startswith("Albert") and not n.endswith("Config")]
