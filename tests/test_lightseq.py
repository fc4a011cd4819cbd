"""LightSeq-style layers, memory planner, GCQ, generation and fake quantisation (CPU)."""
import random

import torch


def test_layers_forward_backward_shapes():
    from oslo_b200.lightseq import (LSCrossEntropyLayer, LSGptEncoderLayer, LSLayerConfig, LSTransformerDecoderLayer,
                                    LSTransformerEmbeddingLayer, LSTransformerEncoderLayer)

    torch.manual_seed(0)
    cfg = LSLayerConfig(hidden_size=32, intermediate_size=64, nhead=4, vocab_size=50, max_seq_len=16, epsilon=0.1)
    emb = LSTransformerEmbeddingLayer(cfg)
    enc, dec, gpt = LSTransformerEncoderLayer(cfg), LSTransformerDecoderLayer(cfg), LSGptEncoderLayer(cfg)
    ids = torch.randint(1, 50, (2, 8))
    pad = torch.zeros(2, 8, dtype=torch.bool)
    pad[1, 6:] = True
    x = emb(ids)
    e = enc(x, pad)
    d = dec(emb(ids), e, pad)
    g = gpt(x)
    assert e.shape == d.shape == g.shape == (2, 8, 32)
    # causal block: output at position t must not depend on later inputs
    x2 = x.clone()
    x2[:, 5:] += 1.0
    assert torch.allclose(gpt(x2)[:, :5], g[:, :5], atol=1e-5)
    head = torch.nn.Linear(32, 50)
    loss, nll = LSCrossEntropyLayer(cfg)(head(d), ids)
    loss.backward()
    assert loss.item() > 0 and nll.item() > 0


def test_memory_planner_no_overlap_and_saves_memory():
    from oslo_b200.lightseq.memory_planner import check, plan

    random.seed(1)
    n = 300
    first = [random.randint(0, 200) for _ in range(n)]
    last = [f + random.randint(0, 30) for f in first]
    sizes = [random.randint(1, 500) * 256 for _ in range(n)]
    offsets, total = plan(sizes, first, last)
    assert check(sizes, first, last, offsets)
    assert total < sum(sizes) / 3
    # tensors alive at the same time need at least their combined size
    peak = max(sum(s for s, f, l in zip(sizes, first, last) if f <= t <= l) for t in range(231))
    assert total >= peak


def test_gcq_single_process_roundtrip():
    from oslo_b200.lightseq import GCQState, quantized_all_reduce

    torch.manual_seed(2)
    g = torch.randn(1000, 64)
    out = quantized_all_reduce(g, GCQState(hidden_size=64, quantile_value=1.0))
    assert (out - g).abs().max() < g.abs().max() / 100


def test_generate_greedy_beam_and_ngram_block():
    from oslo_b200.lightseq import generate
    from oslo_b200.models import GPT2Config, GPT2LMHeadModel

    torch.manual_seed(3)
    m = GPT2LMHeadModel(GPT2Config(vocab_size=40, n_positions=64, n_embd=32, n_layer=1, n_head=4, resid_pdrop=0.0,
                                   embd_pdrop=0.0, attn_pdrop=0.0))
    prompt = torch.randint(0, 40, (2, 4))
    greedy = generate(m, prompt, max_new_tokens=8)
    assert greedy.shape == (2, 12) and torch.equal(greedy[:, :4], prompt)
    beam = generate(m, prompt, max_new_tokens=8, num_beams=3)
    assert beam.shape == (2, 12)
    blocked = generate(m, prompt, max_new_tokens=20, no_repeat_ngram_size=2)
    for row in blocked.tolist():
        bigrams = list(zip(row, row[1:]))
        assert len(bigrams) == len(set(bigrams))
    sampled = generate(m, prompt, max_new_tokens=5, do_sample=True, top_k=5, top_p=0.9)
    assert sampled.shape == (2, 9)


def test_fake_quant_straight_through():
    from oslo_b200.lightseq import QuantLinear

    torch.manual_seed(4)
    q = QuantLinear(16, 8)
    x = torch.randn(4, 16, requires_grad=True)
    y = q(x)
    y.sum().backward()
    ref = torch.nn.functional.linear(x, q.weight, q.bias)
    assert (y - ref).abs().max() < 0.2 and x.grad is not None and q.weight.grad is not None


def test_kv_cache_generation_equals_full_prefix_generation():
    """Greedy and beam decoding with the key / value cache give the same tokens as re-running the whole prefix,
    for every in-tree causal model (learned positions, partial rotary, full rotary), and the cache grows by one
    position per step instead of being rebuilt."""
    from oslo_b200 import models
    from oslo_b200.lightseq import generate
    from oslo_b200.models.config import GPTNeoXConfig
    from oslo_b200.models.gpt_neox import GPTNeoXForCausalLM
    from oslo_b200.ops.attention import DecodeCache, decode_cache

    torch.manual_seed(0)
    built = [
        models.GPT2LMHeadModel(models.GPT2Config(vocab_size=64, n_positions=48, n_embd=32, n_layer=2, n_head=4, resid_pdrop=0.0,
                                                 embd_pdrop=0.0, attn_pdrop=0.0)),
        GPTNeoXForCausalLM(GPTNeoXConfig(vocab_size=64, hidden_size=32, num_hidden_layers=2, num_attention_heads=4,
                                         intermediate_size=64, rotary_pct=0.5, max_position_embeddings=48)),
        models.LlamaForCausalLM(models.LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                                                   num_attention_heads=4, max_position_embeddings=48)),
    ]
    prompt = torch.randint(0, 64, (3, 5))
    for m in built:
        m.eval()
        for kw in (dict(), dict(num_beams=3), dict(no_repeat_ngram_size=2)):
            a = generate(m, prompt, max_new_tokens=10, use_cache=True, **kw)
            b = generate(m, prompt, max_new_tokens=10, use_cache=False, **kw)
            assert torch.equal(a, b), (type(m).__name__, kw)
        # incremental logits equal full-prefix logits, and the cache holds one entry per layer of prompt + steps length
        cache = DecodeCache()
        ids = prompt
        with torch.no_grad():
            for step in range(3):
                cache.begin_forward()
                with decode_cache(cache):
                    inc = m(input_ids=ids[:, cache.offset:]).logits[:, -1]
                cache.advance(ids.shape[1] - cache.offset)
                full = m(input_ids=ids).logits[:, -1]
                assert torch.allclose(inc, full, atol=1e-5), (type(m).__name__, step, (inc - full).abs().max().item())
                ids = torch.cat([ids, full.argmax(-1, keepdim=True)], dim=1)
        assert len(cache.k) == 2 and cache.k[0].shape[1] == prompt.shape[1] + 2


def test_sampling_filter_and_embedding_reference_paths():
    """CPU statements of the LightSeq kernels: nucleus / top-k filtering keeps the right set, sampled tokens come from it,
    the embedding op zeroes padding rows and int8 quantisation round-trips within one step."""
    from oslo_b200.lightseq import filter_logits, ls_dequantize_int8, ls_embedding, ls_quantize_int8, sample_tokens

    torch.manual_seed(0)
    logits = torch.tensor([[4.0, 3.0, 2.0, 1.0, 0.0, -1.0]])
    kept = torch.isfinite(filter_logits(logits, top_k=3, top_p=1.0))[0].tolist()
    assert kept == [True, True, True, False, False, False]
    probs = logits.softmax(-1)[0]
    kept_p = torch.isfinite(filter_logits(logits, top_k=0, top_p=float(probs[0] + probs[1] / 2)))[0].tolist()
    assert kept_p == [True, True, False, False, False, False]  # the smallest prefix whose mass reaches top_p
    draws = torch.cat([sample_tokens(logits.repeat(64, 1), top_k=2) for _ in range(4)])
    assert set(draws.view(-1).tolist()) <= {0, 1} and len(set(draws.view(-1).tolist())) == 2
    emb = torch.randn(10, 16)
    pos = torch.randn(8, 16)
    ids = torch.tensor([[1, 2, 0, 3]])
    out = ls_embedding(ids, emb, pos, step=2, padding_idx=0, scale=4.0)
    assert torch.allclose(out[0, 0], emb[1] * 4.0 + pos[2]) and float(out[0, 2].abs().sum()) == 0.0
    x = torch.randn(1000) * 2
    q, mask = ls_quantize_int8(x, 3.0, return_mask=True)
    back = ls_dequantize_int8(q, 3.0)
    assert q.dtype == torch.int8 and (back - x.clamp(-3, 3)).abs().max() <= 3.0 / 127 / 2 + 1e-6
    assert torch.equal(mask, x.abs() > 3.0)
