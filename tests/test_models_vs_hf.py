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
