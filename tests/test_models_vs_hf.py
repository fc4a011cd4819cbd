"""The in-tree GPT-NeoX, Llama and GPT-2 models against the Hugging Face implementations on the same weights (CPU).

State-dict names follow Hugging Face, so ``load_state_dict`` of a Hugging Face checkpoint must fill every tensor, and
logits must agree for a batch of several rows whose length is shorter than the maximum position (rotary tables and
learned positions are indexed per row, not per flattened token)."""
import warnings

import pytest
import torch

warnings.filterwarnings("ignore")


def _check(ours, theirs, vocab, atol=2e-5):
    res = ours.load_state_dict(theirs.state_dict(), strict=False)
    assert not res.missing_keys, res.missing_keys
    ids = torch.randint(0, vocab, (3, 12), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        a = theirs(input_ids=ids).logits
        b = ours(input_ids=ids).logits
    assert a.shape == b.shape
    assert (a - b).abs().max().item() < atol, (a - b).abs().max().item()


def test_gpt_neox_matches_hugging_face():
    from transformers import GPTNeoXConfig as HC, GPTNeoXForCausalLM as HM

    from oslo_b200.models.config import GPTNeoXConfig
    from oslo_b200.models.gpt_neox import GPTNeoXForCausalLM

    torch.manual_seed(0)
    kw = dict(vocab_size=100, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
              rotary_pct=0.25, max_position_embeddings=32)
    theirs = HM(HC(use_parallel_residual=True, hidden_act="gelu_new", tie_word_embeddings=False, **kw)).eval()
    _check(GPTNeoXForCausalLM(GPTNeoXConfig(**kw)).eval(), theirs, 100)


def test_llama_matches_hugging_face():
    from transformers import LlamaConfig as HC, LlamaForCausalLM as HM

    from oslo_b200.models import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(1)
    kw = dict(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
              max_position_embeddings=32)
    theirs = HM(HC(num_key_value_heads=4, tie_word_embeddings=False, **kw)).eval()
    _check(LlamaForCausalLM(LlamaConfig(**kw)).eval(), theirs, 128)


def test_gpt2_matches_hugging_face():
    from transformers import GPT2Config as HC, GPT2LMHeadModel as HM

    from oslo_b200.models import GPT2Config, GPT2LMHeadModel

    torch.manual_seed(2)
    kw = dict(vocab_size=100, n_positions=32, n_embd=64, n_layer=2, n_head=4, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    theirs = HM(HC(**kw)).eval()
    _check(GPT2LMHeadModel(GPT2Config(**kw)).eval(), theirs, 100)


def test_chunked_head_loss_equals_the_materialised_head_for_the_causal_models():
    from oslo_b200 import models
    from oslo_b200.models.config import GPTNeoXConfig
    from oslo_b200.models.gpt_neox import GPTNeoXForCausalLM

    torch.manual_seed(0)
    cases = [
        (GPTNeoXForCausalLM, GPTNeoXConfig(vocab_size=101, hidden_size=32, num_hidden_layers=2, num_attention_heads=4,
                                           intermediate_size=64, max_position_embeddings=32)),
        (models.GPT2LMHeadModel, models.GPT2Config(vocab_size=101, n_positions=32, n_embd=32, n_layer=2, n_head=4, resid_pdrop=0.0,
                                                   embd_pdrop=0.0, attn_pdrop=0.0, tie_word_embeddings=False)),
        (models.LlamaForCausalLM, models.LlamaConfig(vocab_size=101, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                                                     num_attention_heads=4, max_position_embeddings=32)),
    ]
    ids = torch.randint(0, 101, (3, 17))
    labels = ids.clone()
    labels[1, :4] = -100
    for cls, cfg in cases:
        model = cls(cfg)
        ref = model(input_ids=ids, labels=labels).loss
        ref.backward()
        want = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
        model.zero_grad()
        model.config.chunked_head_loss = 8
        out = model(input_ids=ids, labels=labels)
        assert out.logits is None and torch.allclose(out.loss, ref, atol=1e-5), cls.__name__
        out.loss.backward()
        for n, p in model.named_parameters():
            if n in want:
                assert torch.allclose(p.grad, want[n], atol=2e-5), (cls.__name__, n)


def test_in_tree_checkpoints_load_in_transformers(tmp_path):
    """``save_pretrained`` of an in-tree model writes a directory that the Hugging Face class of the same name loads as is
    (config and state-dict names), and the two give the same logits: moving between the frameworks needs no conversion."""
    transformers = pytest.importorskip("transformers")
    from oslo_b200 import models

    torch.manual_seed(0)
    cases = [
        ("GPT2LMHeadModel", models.GPT2LMHeadModel(models.GPT2Config(vocab_size=100, n_positions=32, n_embd=32, n_layer=2, n_head=4))),
        ("BertForMaskedLM", models.BertForMaskedLM(models.BertConfig(vocab_size=100, hidden_size=32, num_hidden_layers=2,
                                                                      num_attention_heads=4, intermediate_size=64,
                                                                      max_position_embeddings=32))),
        ("T5ForConditionalGeneration", models.T5ForConditionalGeneration(models.T5Config(
            vocab_size=100, d_model=32, d_kv=8, d_ff=64, num_layers=2, num_decoder_layers=2, num_heads=4))),
        ("LlamaForCausalLM", models.LlamaForCausalLM(models.LlamaConfig(vocab_size=100, hidden_size=32, intermediate_size=64,
                                                                        num_hidden_layers=2, num_attention_heads=4,
                                                                        max_position_embeddings=32))),
    ]
    ids = torch.randint(0, 100, (2, 10))
    for name, ours in cases:
        ours.eval()
        path = str(tmp_path / name)
        ours.save_pretrained(path)
        theirs = getattr(transformers, name).from_pretrained(path).eval()
        extra = {"decoder_input_ids": ids[:, :5]} if "T5" in name else {}
        with torch.no_grad():
            assert torch.allclose(ours(input_ids=ids, **extra).logits, theirs(input_ids=ids, **extra).logits, atol=1e-4), name
