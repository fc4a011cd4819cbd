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
