"""In-tree BERT, RoBERTa, ELECTRA, DistilBERT, ALBERT, BART, mBART, T5 and mT5 models.

Each family loads the Hugging Face state dict of a small random model without missing or unexpected keys and reproduces
its outputs and losses (with and without a padding mask); the encoder and the encoder-decoder stacks also reproduce
themselves under 1-D tensor parallelism over two CPU ranks through the built-in name tables."""
import warnings

import pytest
import torch

from dist_utils import run_dist

T = pytest.importorskip("transformers")
warnings.filterwarnings("ignore")

ENC = dict(vocab_size=100, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
           max_position_embeddings=40, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
DISTIL = dict(vocab_size=100, max_position_embeddings=40, n_layers=2, n_heads=4, dim=64, hidden_dim=128, dropout=0.0,
              attention_dropout=0.0, seq_classif_dropout=0.0, qa_dropout=0.0)
ALBERT = dict(vocab_size=100, embedding_size=32, hidden_size=64, num_hidden_layers=3, num_attention_heads=4,
              intermediate_size=128, max_position_embeddings=40, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0,
              classifier_dropout_prob=0.0)
BART = dict(vocab_size=100, max_position_embeddings=40, encoder_layers=2, decoder_layers=2, encoder_ffn_dim=128,
            decoder_ffn_dim=128, encoder_attention_heads=4, decoder_attention_heads=4, d_model=64, dropout=0.0,
            attention_dropout=0.0, activation_dropout=0.0, classifier_dropout=0.0)
T5 = dict(vocab_size=100, d_model=64, d_kv=16, d_ff=128, num_layers=2, num_heads=4, relative_attention_num_buckets=8,
          relative_attention_max_distance=20, dropout_rate=0.0, decoder_start_token_id=0, pad_token_id=0)


def _pair(module, name, cfg_name, kw):
    import importlib

    from oslo_b200.models import config as C

    ours = getattr(importlib.import_module(f"oslo_b200.models.{module}"), name)(getattr(C, cfg_name)(**kw)).eval()
    theirs = getattr(T, name)(getattr(T, cfg_name)(**kw)).eval()
    res = ours.load_state_dict(theirs.state_dict(), strict=False)
    assert not res.missing_keys, res.missing_keys
    assert not res.unexpected_keys, res.unexpected_keys
    return ours, theirs


def _compare(ours, theirs, keys, tol=5e-5, **inputs):
    with torch.no_grad():
        a, b = theirs(**inputs), ours(**inputs)
    mask = inputs.get("attention_mask")
    for k in keys:
        d = (getattr(a, k) - b[k]).abs()
        if mask is not None and d.dim() >= 2 and d.shape[:2] == mask.shape:  # padded positions carry no meaning
            d = d * mask.view(*mask.shape, *([1] * (d.dim() - 2)))
        assert d.max().item() < tol, (type(ours).__name__, k, d.max().item())
    if getattr(a, "loss", None) is not None:
        assert abs(a.loss.item() - b.loss.item()) < 1e-4, (a.loss.item(), b.loss.item())


def _inputs():
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(3, 100, (3, 12), generator=g)
    mask = torch.ones(3, 12, dtype=torch.long)
    mask[1, 8:] = 0
    mask[2, 5:] = 0
    return ids, mask, torch.randint(3, 100, (3, 12), generator=g)


SEQ, TOK = torch.tensor([0, 2, 1]), None
QA = dict(start_positions=torch.tensor([1, 2, 3]), end_positions=torch.tensor([4, 5, 4]))

ENCODER_CASES = [
    ("bert", "BertForMaskedLM", "BertConfig", ENC, ("logits",), "mlm"),
    ("bert", "BertForPreTraining", "BertConfig", ENC, ("prediction_logits", "seq_relationship_logits"), "pretrain"),
    ("bert", "BertForSequenceClassification", "BertConfig", dict(ENC, num_labels=3), ("logits",), "seq"),
    ("bert", "BertForTokenClassification", "BertConfig", dict(ENC, num_labels=5), ("logits",), "tok"),
    ("bert", "BertForQuestionAnswering", "BertConfig", ENC, ("start_logits", "end_logits"), "qa"),
    ("bert", "RobertaForMaskedLM", "RobertaConfig", dict(ENC, pad_token_id=1, type_vocab_size=1), ("logits",), "mlm"),
    ("bert", "RobertaForSequenceClassification", "RobertaConfig", dict(ENC, pad_token_id=1, type_vocab_size=1, num_labels=3),
     ("logits",), "seq"),
    ("bert", "RobertaForQuestionAnswering", "RobertaConfig", dict(ENC, pad_token_id=1, type_vocab_size=1),
     ("start_logits", "end_logits"), "qa"),
    ("bert", "ElectraForMaskedLM", "ElectraConfig", dict(ENC, embedding_size=32), ("logits",), "mlm"),
    ("bert", "ElectraForPreTraining", "ElectraConfig", dict(ENC, embedding_size=32), ("logits",), "disc"),
    ("bert", "ElectraForSequenceClassification", "ElectraConfig", dict(ENC, embedding_size=32, num_labels=3), ("logits",), "seq"),
    ("distilbert", "DistilBertForMaskedLM", "DistilBertConfig", DISTIL, ("logits",), "mlm"),
    ("distilbert", "DistilBertForSequenceClassification", "DistilBertConfig", dict(DISTIL, num_labels=3), ("logits",), "seq"),
    ("distilbert", "DistilBertForQuestionAnswering", "DistilBertConfig", DISTIL, ("start_logits", "end_logits"), "qa"),
    ("albert", "AlbertForMaskedLM", "AlbertConfig", ALBERT, ("logits",), "mlm"),
    ("albert", "AlbertForPreTraining", "AlbertConfig", ALBERT, ("prediction_logits", "sop_logits"), "sop"),
    ("albert", "AlbertForSequenceClassification", "AlbertConfig", dict(ALBERT, num_labels=3), ("logits",), "seq"),
    ("albert", "AlbertForTokenClassification", "AlbertConfig", dict(ALBERT, num_labels=5), ("logits",), "tok"),
]


@pytest.mark.parametrize("module,name,cfg,kw,keys,task", ENCODER_CASES, ids=[c[1] for c in ENCODER_CASES])
def test_encoder_family_matches_hugging_face(module, name, cfg, kw, keys, task):
    torch.manual_seed(0)
    ours, theirs = _pair(module, name, cfg, kw)
    ids, mask, labels = _inputs()
    extra = {"mlm": dict(labels=labels), "seq": dict(labels=SEQ), "qa": QA,
             "tok": dict(labels=torch.randint(0, 5, (3, 12), generator=torch.Generator().manual_seed(3))),
             "pretrain": dict(labels=labels, next_sentence_label=torch.tensor([0, 1, 0])),
             "sop": dict(labels=labels, sentence_order_label=torch.tensor([0, 1, 0])),
             "disc": dict(labels=torch.randint(0, 2, (3, 12), generator=torch.Generator().manual_seed(4)))}[task]
    for m in (None, mask):
        _compare(ours, theirs, keys, input_ids=ids, attention_mask=m, **extra)


SEQ2SEQ_CASES = [
    ("bart", "BartForConditionalGeneration", "BartConfig", BART),
    ("bart", "MBartForConditionalGeneration", "MBartConfig", dict(BART, scale_embedding=True)),
    ("t5", "T5ForConditionalGeneration", "T5Config", T5),
    ("t5", "MT5ForConditionalGeneration", "MT5Config", dict(T5, feed_forward_proj="gated-gelu", tie_word_embeddings=False)),
]


@pytest.mark.parametrize("module,name,cfg,kw", SEQ2SEQ_CASES, ids=[c[1] for c in SEQ2SEQ_CASES])
def test_seq2seq_family_matches_hugging_face(module, name, cfg, kw):
    torch.manual_seed(1)
    ours, theirs = _pair(module, name, cfg, kw)
    ids, mask, labels = _inputs()
    ids[:, -1] = 2
    dec = labels[:, :9].contiguous()
    for m in (None, mask):
        _compare(ours, theirs, ("logits",), tol=1e-4, input_ids=ids, attention_mask=m, decoder_input_ids=dec)
        _compare(ours, theirs, ("logits",), tol=1e-4, input_ids=ids, attention_mask=m, labels=dec)  # decoder inputs from labels
    out = ours.generate(ids[:2], max_new_tokens=4)
    assert out.shape[0] == 2 and 2 <= out.shape[1] <= 5
    # incremental decoding over the key / value cache gives the tokens of full-prefix decoding, greedy and beam, with and
    # without source padding; and the greedy tokens are Hugging Face's
    ours.config.eos_token_id = theirs.config.eos_token_id = -1  # random weights: never stop early, compare every step
    ours.double()  # random weights give near-tied beam candidates: keep cached-vs-full rounding far below the gaps
    for m in (None, mask):
        for beams in (1, 3):
            cached = ours.generate(ids, m, max_new_tokens=7, num_beams=beams, use_cache=True)
            full = ours.generate(ids, m, max_new_tokens=7, num_beams=beams, use_cache=False)
            assert torch.equal(cached, full), (name, beams, m is not None)
    ours.float()
    from oslo_b200.models.modeling_utils import Seq2SeqCache, active_seq2seq_cache

    assert active_seq2seq_cache() is None  # the cache does not outlive generate()
    cache = Seq2SeqCache()
    assert cache.offset == 0 and not cache.self_kv
    if name in ("BartForConditionalGeneration", "T5ForConditionalGeneration"):  # (mBART's generation config forces other tokens)
        hf = theirs.generate(input_ids=ids, attention_mask=mask, max_new_tokens=7, num_beams=1, do_sample=False, min_length=0)
        mine = ours.generate(ids, mask, max_new_tokens=7)
        assert torch.equal(mine[:, : hf.shape[1]], hf[:, : mine.shape[1]]), name


def test_bart_heads_match_hugging_face():
    torch.manual_seed(2)
    ids, mask, _ = _inputs()
    ids[:, -1] = 2
    ours, theirs = _pair("bart", "BartForSequenceClassification", "BartConfig", dict(BART, num_labels=3))
    _compare(ours, theirs, ("logits",), input_ids=ids, labels=SEQ)
    ours, theirs = _pair("bart", "BartForQuestionAnswering", "BartConfig", BART)
    _compare(ours, theirs, ("start_logits", "end_logits"), input_ids=ids, **QA)
    from oslo_b200.models.bart import BartForCausalLM
    from oslo_b200.models.config import BartConfig

    ours = BartForCausalLM(BartConfig(**BART)).eval()
    theirs = T.BartForCausalLM(T.BartConfig(is_decoder=True, is_encoder_decoder=False, **BART)).eval()
    res = ours.load_state_dict(theirs.state_dict(), strict=False)
    assert not res.missing_keys and not res.unexpected_keys, res
    _compare(ours, theirs, ("logits",), input_ids=ids, labels=ids)


def test_bias_act_reference_forms():
    from oslo_b200.ops.activation import bias_act

    x, b = torch.randn(4, 16), torch.randn(16)
    assert torch.allclose(bias_act(x, b, "gelu"), torch.nn.functional.gelu(x + b))
    assert torch.allclose(bias_act(x, b, "gelu_new"), torch.nn.functional.gelu(x + b, approximate="tanh"))
    assert torch.allclose(bias_act(x, None, "relu"), torch.relu(x))
    with pytest.raises(ValueError):
        bias_act(x, b, "swish")


def _tp_worker(rank, world, module, name, cfg, kw, seq2seq):
    import importlib

    import oslo_b200
    from oslo_b200 import ParallelContext
    from oslo_b200.models import config as C
    from oslo_b200.parallel import TensorParallel

    pc = ParallelContext.from_torch(tensor_parallel_size=world, backend="gloo", seed=0)
    cls = getattr(importlib.import_module(f"oslo_b200.models.{module}"), name)
    torch.manual_seed(0)
    ref = cls(getattr(C, cfg)(**kw)).eval()
    torch.manual_seed(0)
    model = cls(getattr(C, cfg)(**kw)).eval()
    wrapped = TensorParallel(model, pc)
    oslo_b200.ready(wrapped, pc)
    ids, mask, labels = _inputs()
    inputs = dict(input_ids=ids, attention_mask=mask)
    if seq2seq:
        inputs["decoder_input_ids"] = labels[:, :9].contiguous()
    with torch.no_grad():
        want, got = ref(**inputs).logits, wrapped(**inputs).logits
        if got.shape[-1] != want.shape[-1]:  # in-tree heads keep the vocabulary sharded for the vocab-parallel loss
            import torch.distributed as dist

            parts = [torch.empty_like(got) for _ in range(world)]
            dist.all_gather(parts, got.contiguous())
            got = torch.cat(parts, dim=-1)[..., : want.shape[-1]]
        tgt = labels[:, :9].contiguous() if seq2seq else labels
        want_loss = ref(**inputs, labels=tgt).loss
        got_loss = wrapped(**inputs, labels=tgt).loss
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.allclose(got, want, rtol=1e-4, atol=2e-5), (got - want).abs().max()
    assert abs(want_loss.item() - got_loss.item()) < 1e-4, (want_loss.item(), got_loss.item())
    assert len([n for n, p in model.named_parameters() if hasattr(p, "oslo_shard")]) >= 8
    pc.destroy()


TP_CASES = [("bert", "BertForMaskedLM", "BertConfig", ENC, False),
            ("bert", "ElectraForMaskedLM", "ElectraConfig", dict(ENC, embedding_size=32), False),
            ("distilbert", "DistilBertForMaskedLM", "DistilBertConfig", DISTIL, False),
            ("albert", "AlbertForMaskedLM", "AlbertConfig", ALBERT, False),
            ("bart", "BartForConditionalGeneration", "BartConfig", BART, True),
            ("t5", "T5ForConditionalGeneration", "T5Config", T5, True)]


@pytest.mark.parametrize("module,name,cfg,kw,seq2seq", TP_CASES, ids=[c[1] for c in TP_CASES])
def test_in_tree_family_tensor_parallel_1d(module, name, cfg, kw, seq2seq):
    run_dist(_tp_worker, 2, module, name, cfg, kw, seq2seq, timeout=600)
