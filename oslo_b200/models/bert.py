"""BERT-style post-LayerNorm encoders: BERT, RoBERTa and ELECTRA share one layer stack here.

Module and state-dict names follow the Hugging Face classes of the same names (``bert.encoder.layer.N.attention.self.query``
and so on), so their checkpoints load directly and the built-in tensor-parallel name tables apply unchanged.  The layers
run on the fused ops: bias + activation in one pass, bias + dropout + residual in one pass, fused LayerNorm, and the
tcgen05 attention kernel when no padding mask is given (with a mask the scores go through the masked softmax path).
Dropout on the attention probabilities is not applied (the fused attention keeps no probability matrix).

Parity: oslo/transformers/models/bert/modeling_bert.py, roberta/modeling_roberta.py, electra/modeling_electra.py.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

import oslo_b200.nn as onn
from oslo_b200.nn import functional as OF

from .config import BertConfig, ElectraConfig, RobertaConfig
from .heads import classification_loss, qa_loss
from .losses import token_lm_loss
from .modeling_utils import ModelOutput, PreTrainedModel, additive_mask


class BertEmbeddings(nn.Module):
    """Word + position + token-type embeddings, LayerNorm, dropout.  ``padding_offset`` (RoBERTa) numbers positions from
    ``pad_token_id + 1`` and skips padding tokens."""

    def __init__(self, config, embedding_size=None, padding_offset=False):
        super().__init__()
        e = embedding_size or config.hidden_size
        self.word_embeddings = nn.Embedding(config.vocab_size, e, padding_idx=config.pad_token_id)
        self.position_embeddings = nn.Embedding(config.max_position_embeddings, e,
                                                padding_idx=config.pad_token_id if padding_offset else None)
        self.token_type_embeddings = nn.Embedding(config.type_vocab_size, e)
        self.LayerNorm = onn.FusedLayerNorm(e, eps=config.layer_norm_eps)
        self.dropout = nn.Dropout(config.hidden_dropout_prob)
        self.padding_offset, self.pad_token_id = padding_offset, config.pad_token_id

    def forward(self, input_ids, token_type_ids=None, position_ids=None):
        b, s = input_ids.shape
        if position_ids is None:
            if self.padding_offset:
                keep = input_ids.ne(self.pad_token_id).long()
                position_ids = torch.cumsum(keep, dim=1) * keep + self.pad_token_id
            else:
                position_ids = torch.arange(s, device=input_ids.device).unsqueeze(0)
        if token_type_ids is None:
            token_type_ids = torch.zeros_like(input_ids)
        x = self.word_embeddings(input_ids) + self.token_type_embeddings(token_type_ids) + self.position_embeddings(position_ids)
        return self.dropout(self.LayerNorm(x))


class BertSelfAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.num_attention_heads = config.num_attention_heads
        self.attention_head_size = config.hidden_size // config.num_attention_heads
        self.all_head_size = config.hidden_size
        self.query = onn.Linear(config.hidden_size, self.all_head_size)
        self.key = onn.Linear(config.hidden_size, self.all_head_size)
        self.value = onn.Linear(config.hidden_size, self.all_head_size)

    def forward(self, hidden_states, mask=None):
        b, s, _ = hidden_states.shape
        hd = self.attention_head_size
        q, k, v = (lin(hidden_states).unflatten(-1, (-1, hd)) for lin in (self.query, self.key, self.value))
        return OF.attention(q, k, v, causal=False, mask=mask)


class BertSelfOutput(nn.Module):
    def __init__(self, config, in_features=None):
        super().__init__()
        self.dense = onn.Linear(in_features or config.hidden_size, config.hidden_size, skip_bias_add=True)
        self.LayerNorm = onn.FusedLayerNorm(config.hidden_size, eps=config.layer_norm_eps)
        self.p = config.hidden_dropout_prob

    def forward(self, hidden_states, residual):
        h, bias = self.dense(hidden_states)
        return self.LayerNorm(OF.bias_dropout_add(h, bias, residual, self.p, self.training))


class BertAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.self = BertSelfAttention(config)
        self.output = BertSelfOutput(config)

    def forward(self, hidden_states, mask=None):
        return self.output(self.self(hidden_states, mask), hidden_states)


class BertIntermediate(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = onn.Linear(config.hidden_size, config.intermediate_size, skip_bias_add=True)
        self.act = config.hidden_act

    def forward(self, hidden_states):
        h, bias = self.dense(hidden_states)
        return OF.bias_act(h, bias, self.act)


class BertOutput(BertSelfOutput):
    def __init__(self, config):
        super().__init__(config, in_features=config.intermediate_size)


class BertLayer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.attention = BertAttention(config)
        self.intermediate = BertIntermediate(config)
        self.output = BertOutput(config)

    def forward(self, hidden_states, mask=None):
        a = self.attention(hidden_states, mask)
        return self.output(self.intermediate(a), a)


class BertEncoder(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.layer = nn.ModuleList([BertLayer(config) for _ in range(config.num_hidden_layers)])
        self.gradient_checkpointing = False

    def forward(self, hidden_states, mask=None):
        for layer in self.layer:
            if self.gradient_checkpointing and self.training:
                hidden_states = torch.utils.checkpoint.checkpoint(layer, hidden_states, mask, use_reentrant=False)
            else:
                hidden_states = layer(hidden_states, mask)
        return hidden_states


class BertPooler(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = onn.Linear(config.hidden_size, config.hidden_size)

    def forward(self, hidden_states):
        return torch.tanh(self.dense(hidden_states[:, 0]))


class BertPreTrainedModel(PreTrainedModel):
    config_class = BertConfig
    base_model_prefix = "bert"

    def get_input_embeddings(self):
        return getattr(self, self.base_model_prefix, self).embeddings.word_embeddings

    def gradient_checkpointing_enable(self):
        getattr(self, self.base_model_prefix, self).encoder.gradient_checkpointing = True


class BertModel(BertPreTrainedModel):
    padding_offset = False

    def __init__(self, config, add_pooling_layer=True):
        super().__init__(config)
        self.embeddings = BertEmbeddings(config, padding_offset=self.padding_offset)
        self.encoder = BertEncoder(config)
        self.pooler = BertPooler(config) if add_pooling_layer else None
        self.post_init()

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, position_ids=None, **unused):
        x = self.embeddings(input_ids, token_type_ids, position_ids)
        x = self.encoder(x, additive_mask(attention_mask, torch.float32))
        return ModelOutput(last_hidden_state=x, pooler_output=self.pooler(x) if self.pooler is not None else None)


class BertPredictionHeadTransform(nn.Module):
    def __init__(self, config, size=None):
        super().__init__()
        size = size or config.hidden_size
        self.dense = onn.Linear(config.hidden_size, size, skip_bias_add=True)
        self.act = config.hidden_act
        self.LayerNorm = onn.FusedLayerNorm(size, eps=config.layer_norm_eps)

    def forward(self, hidden_states):
        h, bias = self.dense(hidden_states)
        return self.LayerNorm(OF.bias_act(h, bias, self.act))


class BertLMPredictionHead(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.transform = BertPredictionHeadTransform(config)
        self.decoder = onn.Linear(config.hidden_size, config.vocab_size, bias=True)
        self.bias = self.decoder.bias  # the same tensor under both names, as in Hugging Face checkpoints

    def forward(self, hidden_states):
        return self.decoder(self.transform(hidden_states))


class BertOnlyMLMHead(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.predictions = BertLMPredictionHead(config)

    def forward(self, x):
        return self.predictions(x)


class BertPreTrainingHeads(BertOnlyMLMHead):
    def __init__(self, config):
        super().__init__(config)
        self.seq_relationship = onn.Linear(config.hidden_size, 2)


def _mlm_output(model, logits, labels, **extra):
    loss = None
    if labels is not None:
        res = token_lm_loss(model, logits, labels)
        loss, logits = res.value, (None if res.consumed_logits else logits)
    return loss, logits


class BertForMaskedLM(BertPreTrainedModel):
    def __init__(self, config):
        super().__init__(config)
        self.bert = BertModel(config, add_pooling_layer=False)
        self.cls = BertOnlyMLMHead(config)
        self.post_init()

    def get_output_embeddings(self):
        return self.cls.predictions.decoder

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, position_ids=None, labels=None, **unused):
        x = self.bert(input_ids, attention_mask, token_type_ids, position_ids).last_hidden_state
        loss, logits = _mlm_output(self, self.cls(x), labels)
        return ModelOutput(loss=loss, logits=logits)


class BertForPreTraining(BertPreTrainedModel):
    """Masked-LM plus next-sentence heads; the loss is their sum when both label sets are given."""

    def __init__(self, config):
        super().__init__(config)
        self.bert = BertModel(config)
        self.cls = BertPreTrainingHeads(config)
        self.post_init()

    def get_output_embeddings(self):
        return self.cls.predictions.decoder

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, position_ids=None, labels=None,
                next_sentence_label=None, **unused):
        out = self.bert(input_ids, attention_mask, token_type_ids, position_ids)
        logits = self.cls.predictions(out.last_hidden_state)
        rel = self.cls.seq_relationship(out.pooler_output)
        loss = None
        if labels is not None and next_sentence_label is not None:
            mlm = F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), labels.reshape(-1), ignore_index=-100)
            loss = mlm + F.cross_entropy(rel.float(), next_sentence_label.view(-1))
        return ModelOutput(loss=loss, prediction_logits=logits, seq_relationship_logits=rel)


class BertForNextSentencePrediction(BertPreTrainedModel):
    def __init__(self, config):
        super().__init__(config)
        self.bert = BertModel(config)
        self.cls = nn.Module()
        self.cls.seq_relationship = onn.Linear(config.hidden_size, 2)
        self.post_init()

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, position_ids=None, labels=None, **unused):
        rel = self.cls.seq_relationship(self.bert(input_ids, attention_mask, token_type_ids, position_ids).pooler_output)
        loss = F.cross_entropy(rel.float(), labels.view(-1)) if labels is not None else None
        return ModelOutput(loss=loss, logits=rel)


class SentenceHead(nn.Module):
    """``dense -> act -> out_proj`` on the first token (RoBERTa: tanh, ELECTRA: gelu)."""

    def __init__(self, config, act):
        super().__init__()
        self.dense = onn.Linear(config.hidden_size, config.hidden_size)
        p = config.classifier_dropout if getattr(config, "classifier_dropout", None) is not None else config.hidden_dropout_prob
        self.dropout = nn.Dropout(p)
        self.out_proj = onn.Linear(config.hidden_size, config.num_labels)
        self.act = act

    def forward(self, features):
        x = self.dropout(features[:, 0])
        x = self.dense(x)
        x = torch.tanh(x) if self.act == "tanh" else F.gelu(x)
        return self.out_proj(self.dropout(x))


def _classifier_dropout(config):
    p = getattr(config, "classifier_dropout", None)
    return nn.Dropout(p if p is not None else config.hidden_dropout_prob)


def make_task_models(prefix: str, base_cls, pretrained_cls, two_layer_head=None, module=None):
    """Build ``<Prefix>ForSequenceClassification / TokenClassification / MultipleChoice / QuestionAnswering`` for an
    encoder class; returns them by name."""
    attr = pretrained_cls.base_model_prefix

    def base(self, config, pooled):
        kw = {"add_pooling_layer": pooled} if "add_pooling_layer" in base_cls.__init__.__code__.co_varnames else {}
        setattr(self, attr, base_cls(config, **kw))

    def encode(self, input_ids, attention_mask, token_type_ids, position_ids):
        return getattr(self, attr)(input_ids, attention_mask=attention_mask, token_type_ids=token_type_ids,
                                   position_ids=position_ids)

    class ForSequenceClassification(pretrained_cls):
        def __init__(self, config):
            super().__init__(config)
            self.num_labels = config.num_labels
            base(self, config, two_layer_head is None)
            if two_layer_head is None:
                self.dropout = _classifier_dropout(config)
                self.classifier = onn.Linear(config.hidden_size, config.num_labels)
            else:
                self.classifier = SentenceHead(config, two_layer_head)
            self.post_init()

        def forward(self, input_ids, attention_mask=None, token_type_ids=None, position_ids=None, labels=None, **unused):
            out = encode(self, input_ids, attention_mask, token_type_ids, position_ids)
            if two_layer_head is None:
                logits = self.classifier(self.dropout(out.pooler_output))
            else:
                logits = self.classifier(out.last_hidden_state)
            return ModelOutput(loss=classification_loss(logits, labels, self.num_labels), logits=logits)

    class ForTokenClassification(pretrained_cls):
        def __init__(self, config):
            super().__init__(config)
            self.num_labels = config.num_labels
            base(self, config, False)
            self.dropout = _classifier_dropout(config)
            self.classifier = onn.Linear(config.hidden_size, config.num_labels)
            self.post_init()

        def forward(self, input_ids, attention_mask=None, token_type_ids=None, position_ids=None, labels=None, **unused):
            x = encode(self, input_ids, attention_mask, token_type_ids, position_ids).last_hidden_state
            logits = self.classifier(self.dropout(x))
            loss = None
            if labels is not None:
                loss = F.cross_entropy(logits.reshape(-1, self.num_labels).float(), labels.reshape(-1), ignore_index=-100)
            return ModelOutput(loss=loss, logits=logits)

    class ForMultipleChoice(pretrained_cls):
        def __init__(self, config):
            super().__init__(config)
            base(self, config, two_layer_head is None)
            self.dropout = _classifier_dropout(config)
            if two_layer_head is not None:
                self.sequence_summary = nn.Module()
                self.sequence_summary.summary = onn.Linear(config.hidden_size, config.hidden_size)
            self.classifier = onn.Linear(config.hidden_size, 1)
            self.post_init()

        def forward(self, input_ids, attention_mask=None, token_type_ids=None, position_ids=None, labels=None, **unused):
            n = input_ids.shape[1]
            flat = lambda t: t.reshape(-1, t.shape[-1]) if t is not None else None  # noqa: E731
            out = encode(self, flat(input_ids), flat(attention_mask), flat(token_type_ids), flat(position_ids))
            if two_layer_head is None:
                pooled = out.pooler_output
            else:
                pooled = F.gelu(self.sequence_summary.summary(out.last_hidden_state[:, 0]))
            logits = self.classifier(self.dropout(pooled)).view(-1, n)
            loss = F.cross_entropy(logits.float(), labels) if labels is not None else None
            return ModelOutput(loss=loss, logits=logits)

    class ForQuestionAnswering(pretrained_cls):
        def __init__(self, config):
            super().__init__(config)
            base(self, config, False)
            self.qa_outputs = onn.Linear(config.hidden_size, 2)
            self.post_init()

        def forward(self, input_ids, attention_mask=None, token_type_ids=None, position_ids=None, start_positions=None,
                    end_positions=None, **unused):
            x = encode(self, input_ids, attention_mask, token_type_ids, position_ids).last_hidden_state
            start, end = (t.squeeze(-1).contiguous() for t in self.qa_outputs(x).split(1, dim=-1))
            return ModelOutput(loss=qa_loss(start, end, start_positions, end_positions), start_logits=start, end_logits=end)

    out = {}
    for cls in (ForSequenceClassification, ForTokenClassification, ForMultipleChoice, ForQuestionAnswering):
        cls.__name__ = cls.__qualname__ = prefix + cls.__name__
        if module is not None:
            cls.__module__ = module
        out[cls.__name__] = cls
    return out


globals().update(make_task_models("Bert", BertModel, BertPreTrainedModel, module=__name__))


# ----------------------------------------------------------------------------------------------------- RoBERTa
class RobertaPreTrainedModel(BertPreTrainedModel):
    config_class = RobertaConfig
    base_model_prefix = "roberta"


class RobertaModel(BertModel, RobertaPreTrainedModel):
    padding_offset = True


class RobertaLMHead(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = onn.Linear(config.hidden_size, config.hidden_size, skip_bias_add=True)
        self.layer_norm = onn.FusedLayerNorm(config.hidden_size, eps=config.layer_norm_eps)
        self.decoder = onn.Linear(config.hidden_size, config.vocab_size)
        self.bias = self.decoder.bias

    def forward(self, features):
        h, bias = self.dense(features)
        return self.decoder(self.layer_norm(OF.bias_act(h, bias, "gelu")))


class RobertaForMaskedLM(RobertaPreTrainedModel):
    def __init__(self, config):
        super().__init__(config)
        self.roberta = RobertaModel(config, add_pooling_layer=False)
        self.lm_head = RobertaLMHead(config)
        self.post_init()

    def get_output_embeddings(self):
        return self.lm_head.decoder

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, position_ids=None, labels=None, **unused):
        x = self.roberta(input_ids, attention_mask, token_type_ids, position_ids).last_hidden_state
        loss, logits = _mlm_output(self, self.lm_head(x), labels)
        return ModelOutput(loss=loss, logits=logits)


class RobertaForCausalLM(RobertaForMaskedLM):
    """Left-to-right use of the encoder stack (the attention stays bidirectional unless a 4-D mask is passed, as in the
    reference's copy when ``is_decoder`` is unset); labels are shifted by one position."""

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, position_ids=None, labels=None, **unused):
        from .losses import shift_labels

        return super().forward(input_ids, attention_mask, token_type_ids, position_ids,
                               labels=shift_labels(labels) if labels is not None else None)


globals().update(make_task_models("Roberta", RobertaModel, RobertaPreTrainedModel, two_layer_head="tanh", module=__name__))


# ----------------------------------------------------------------------------------------------------- ELECTRA
class ElectraPreTrainedModel(BertPreTrainedModel):
    config_class = ElectraConfig
    base_model_prefix = "electra"


class ElectraModel(ElectraPreTrainedModel):
    def __init__(self, config):
        super().__init__(config)
        self.embeddings = BertEmbeddings(config, embedding_size=config.embedding_size)
        if config.embedding_size != config.hidden_size:
            self.embeddings_project = onn.Linear(config.embedding_size, config.hidden_size)
        self.encoder = BertEncoder(config)
        self.post_init()

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, position_ids=None, **unused):
        x = self.embeddings(input_ids, token_type_ids, position_ids)
        if hasattr(self, "embeddings_project"):
            x = self.embeddings_project(x)
        return ModelOutput(last_hidden_state=self.encoder(x, additive_mask(attention_mask, torch.float32)))


class ElectraGeneratorPredictions(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.LayerNorm = onn.FusedLayerNorm(config.embedding_size, eps=config.layer_norm_eps)
        self.dense = onn.Linear(config.hidden_size, config.embedding_size, skip_bias_add=True)

    def forward(self, x):
        h, bias = self.dense(x)
        return self.LayerNorm(OF.bias_act(h, bias, "gelu"))


class ElectraForMaskedLM(ElectraPreTrainedModel):
    """The generator: masked-LM head over the embedding size, tied to the word embeddings."""

    def __init__(self, config):
        super().__init__(config)
        self.electra = ElectraModel(config)
        self.generator_predictions = ElectraGeneratorPredictions(config)
        self.generator_lm_head = onn.Linear(config.embedding_size, config.vocab_size)
        self.post_init()

    def get_output_embeddings(self):
        return self.generator_lm_head

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, position_ids=None, labels=None, **unused):
        x = self.electra(input_ids, attention_mask, token_type_ids, position_ids).last_hidden_state
        loss, logits = _mlm_output(self, self.generator_lm_head(self.generator_predictions(x)), labels)
        return ModelOutput(loss=loss, logits=logits)


class ElectraDiscriminatorPredictions(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = onn.Linear(config.hidden_size, config.hidden_size, skip_bias_add=True)
        self.dense_prediction = onn.Linear(config.hidden_size, 1)
        self.act = config.hidden_act

    def forward(self, x):
        h, bias = self.dense(x)
        return self.dense_prediction(OF.bias_act(h, bias, self.act)).squeeze(-1)


class ElectraForPreTraining(ElectraPreTrainedModel):
    """The discriminator: a per-token real / replaced logit with a binary cross-entropy over non-padding tokens."""

    def __init__(self, config):
        super().__init__(config)
        self.electra = ElectraModel(config)
        self.discriminator_predictions = ElectraDiscriminatorPredictions(config)
        self.post_init()

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, position_ids=None, labels=None, **unused):
        x = self.electra(input_ids, attention_mask, token_type_ids, position_ids).last_hidden_state
        logits = self.discriminator_predictions(x)
        loss = None
        if labels is not None:
            if attention_mask is not None:
                keep = attention_mask.reshape(-1) == 1
                loss = F.binary_cross_entropy_with_logits(logits.reshape(-1)[keep].float(), labels.reshape(-1)[keep].float())
            else:
                loss = F.binary_cross_entropy_with_logits(logits.float(), labels.float())
        return ModelOutput(loss=loss, logits=logits)


globals().update(make_task_models("Electra", ElectraModel, ElectraPreTrainedModel, two_layer_head="gelu", module=__name__))

__all__ = [n for n in globals() if n.startswith(("Bert", "Roberta", "Electra")) and not n.endswith("Config")]
