"""TensorParallel on stock Hugging Face models (random init, no network): 1-D TP over 2 CPU ranks reproduces the
unsharded logits, and the merged checkpoint equals the original weights."""
import os
import tempfile

import pytest
import torch

from dist_utils import run_dist

transformers = pytest.importorskip("transformers")


def _build(kind):
    torch.manual_seed(0)
    if kind == "gpt2":
        from transformers import GPT2Config, GPT2LMHeadModel

        return GPT2LMHeadModel(GPT2Config(vocab_size=100, n_positions=32, n_embd=32, n_layer=2, n_head=4, resid_pdrop=0.0,
                                          embd_pdrop=0.0, attn_pdrop=0.0)).eval()
    if kind == "bert":
        from transformers import BertConfig, BertForMaskedLM

        return BertForMaskedLM(BertConfig(vocab_size=100, hidden_size=32, num_hidden_layers=2, num_attention_heads=4,
                                          intermediate_size=64, max_position_embeddings=32, hidden_dropout_prob=0.0,
                                          attention_probs_dropout_prob=0.0)).eval()
    if kind == "gpt_neox":
        from transformers import GPTNeoXConfig, GPTNeoXForCausalLM

        return GPTNeoXForCausalLM(GPTNeoXConfig(vocab_size=100, hidden_size=32, num_hidden_layers=2, num_attention_heads=4,
                                                intermediate_size=64, max_position_embeddings=32, hidden_dropout=0.0,
                                                attention_dropout=0.0)).eval()
    if kind == "roberta":
        from transformers import RobertaConfig, RobertaForMaskedLM

        return RobertaForMaskedLM(RobertaConfig(vocab_size=100, hidden_size=32, num_hidden_layers=2, num_attention_heads=4,
                                                intermediate_size=64, max_position_embeddings=40, hidden_dropout_prob=0.0,
                                                attention_probs_dropout_prob=0.0)).eval()
    if kind == "distilbert":
        from transformers import DistilBertConfig, DistilBertForMaskedLM

        return DistilBertForMaskedLM(DistilBertConfig(vocab_size=100, dim=32, n_layers=2, n_heads=4, hidden_dim=64,
                                                      max_position_embeddings=32, dropout=0.0, attention_dropout=0.0)).eval()
    if kind == "electra":
        from transformers import ElectraConfig, ElectraForMaskedLM

        return ElectraForMaskedLM(ElectraConfig(vocab_size=100, embedding_size=32, hidden_size=32, num_hidden_layers=2,
                                                num_attention_heads=4, intermediate_size=64, max_position_embeddings=32,
                                                hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)).eval()
    if kind == "albert":
        from transformers import AlbertConfig, AlbertForMaskedLM

        return AlbertForMaskedLM(AlbertConfig(vocab_size=100, embedding_size=16, hidden_size=32, num_hidden_layers=2,
                                              num_attention_heads=4, intermediate_size=64, max_position_embeddings=32,
                                              hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)).eval()
    if kind == "llama":
        from transformers import LlamaConfig, LlamaForCausalLM

        return LlamaForCausalLM(LlamaConfig(vocab_size=100, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                                            num_attention_heads=4, max_position_embeddings=32)).eval()
    if kind == "opt":
        from transformers import OPTConfig, OPTForCausalLM

        return OPTForCausalLM(OPTConfig(vocab_size=100, hidden_size=32, ffn_dim=64, num_hidden_layers=2, num_attention_heads=4,
                                        max_position_embeddings=32, word_embed_proj_dim=32, dropout=0.0)).eval()
    if kind == "gptj":
        from transformers import GPTJConfig, GPTJForCausalLM

        return GPTJForCausalLM(GPTJConfig(vocab_size=100, n_positions=32, n_embd=32, n_layer=2, n_head=4, rotary_dim=4, resid_pdrop=0.0,
                                          embd_pdrop=0.0, attn_pdrop=0.0)).eval()
    if kind == "gpt_neo":
        from transformers import GPTNeoConfig, GPTNeoForCausalLM

        return GPTNeoForCausalLM(GPTNeoConfig(vocab_size=100, max_position_embeddings=32, hidden_size=32, num_layers=2, num_heads=4,
                                              attention_types=[[["global", "local"], 1]], window_size=8, resid_dropout=0.0,
                                              embed_dropout=0.0, attention_dropout=0.0)).eval()
    if kind == "t5":
        from transformers import T5Config, T5ForConditionalGeneration

        return T5ForConditionalGeneration(T5Config(vocab_size=100, d_model=32, d_kv=8, d_ff=64, num_layers=2, num_decoder_layers=2,
                                                   num_heads=4, dropout_rate=0.0, decoder_start_token_id=0)).eval()
    if kind == "bart":
        from transformers import BartConfig, BartForConditionalGeneration

        return BartForConditionalGeneration(BartConfig(vocab_size=100, d_model=32, encoder_layers=2, decoder_layers=2,
                                                       encoder_attention_heads=4, decoder_attention_heads=4, encoder_ffn_dim=64,
                                                       decoder_ffn_dim=64, max_position_embeddings=32, dropout=0.0,
                                                       attention_dropout=0.0, activation_dropout=0.0)).eval()
    if kind == "blenderbot":
        from transformers import BlenderbotConfig, BlenderbotForConditionalGeneration

        return BlenderbotForConditionalGeneration(BlenderbotConfig(
            vocab_size=100, d_model=32, encoder_layers=2, decoder_layers=2, encoder_attention_heads=4, decoder_attention_heads=4,
            encoder_ffn_dim=64, decoder_ffn_dim=64, max_position_embeddings=32, dropout=0.0, attention_dropout=0.0,
            activation_dropout=0.0)).eval()
    if kind == "vit":
        from transformers import ViTConfig, ViTForImageClassification

        return ViTForImageClassification(ViTConfig(hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
                                                   image_size=16, patch_size=8, num_labels=6, hidden_dropout_prob=0.0,
                                                   attention_probs_dropout_prob=0.0)).eval()
    if kind in ("bert_cls", "bert_qa"):
        from transformers import BertConfig, BertForQuestionAnswering, BertForSequenceClassification

        cfg = BertConfig(vocab_size=100, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
                         max_position_embeddings=32, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0,
                         num_labels=3 if kind == "bert_cls" else 2)
        return (BertForSequenceClassification if kind == "bert_cls" else BertForQuestionAnswering)(cfg).eval()
    raise KeyError(kind)


def _inputs(kind):
    ids = torch.randint(0, 100, (2, 12), generator=torch.Generator().manual_seed(1))
    if kind == "vit":
        return {"pixel_values": torch.randn(2, 3, 16, 16, generator=torch.Generator().manual_seed(1))}
    if kind in ("t5", "bart", "blenderbot"):
        return {"input_ids": ids, "decoder_input_ids": ids[:, :7].contiguous()}
    return {"input_ids": ids}


def _worker(rank, world, kind, tmp):
    import oslo_b200
    from oslo_b200 import ParallelContext
    from oslo_b200.parallel import TensorParallel

    pc = ParallelContext.from_torch(tensor_parallel_size=world, backend="gloo", seed=0)
    ref = _build(kind)
    model = _build(kind)
    state = {k: v.clone() for k, v in ref.state_dict().items()}
    wrapped = TensorParallel(model, pc)
    oslo_b200.ready(wrapped, pc)
    feed = _inputs(kind)
    with torch.no_grad():
        want = ref(**feed).logits
        got = wrapped(**feed).logits
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-5), (got - want).abs().max()
    sharded = [n for n, p in model.named_parameters() if hasattr(p, "oslo_shard")]
    assert len(sharded) >= 8, sharded
    wrapped.save_pretrained(tmp, merge_checkpoints=True)
    if rank == 0:
        merged = torch.load(os.path.join(tmp, "pytorch_model.bin"))
        for k, v in state.items():
            if k in merged:
                assert torch.equal(merged[k], v), k
    pc.destroy()


@pytest.mark.parametrize("kind", ["gpt2", "bert", "gpt_neox", "distilbert", "electra", "albert", "llama", "opt", "gptj",
                                  "gpt_neo", "t5", "bart", "vit"])  # roberta and blenderbot run in the N-D cases below
def test_hf_model_tensor_parallel_1d(kind):
    with tempfile.TemporaryDirectory() as tmp:
        run_dist(_worker, 2, kind, tmp, timeout=600)


def _nd_worker(rank, world, kind, mode, depth):
    """Stock Hugging Face models under the 2-D / 2.5-D / 3-D layouts: same outputs as the unsharded model.  Exercises what
    the 1-D layout never needs: tables shared by an encoder and a decoder under several names, embedding subclasses with
    their own forward (scaled words, learned positions), linears the mapping does not name, task heads with a handful of
    classes, and models whose first hidden state does not come from a token table."""
    import oslo_b200
    from oslo_b200 import ParallelContext, ParallelMode
    from oslo_b200.parallel import TensorParallel

    layout = {"2d": ParallelMode.TENSOR_2D, "2.5d": ParallelMode.TENSOR_2P5D, "3d": ParallelMode.TENSOR_3D}[mode]
    pc = ParallelContext.from_torch(tensor_parallel_size=world, tensor_parallel_mode=layout, tensor_parallel_depth=depth,
                                    backend="gloo", seed=0)
    ref = _build(kind)
    model = _build(kind)
    wrapped = TensorParallel(model, pc)
    oslo_b200.ready(wrapped, pc)
    feed = {k: torch.cat([v, v]) for k, v in _inputs("bert" if kind.startswith("bert_") else kind).items()}  # batch 4
    with torch.no_grad():
        a, b = ref(**feed), wrapped(**feed)
    for key in ("logits", "start_logits", "end_logits"):
        if hasattr(a, key) and getattr(a, key) is not None:
            want, got = getattr(a, key), getattr(b, key)
            assert got.shape == want.shape, (key, got.shape, want.shape)
            assert torch.allclose(got, want, rtol=1e-4, atol=1e-5), (key, (got - want).abs().max())
    pc.destroy()


ND_CASES = [(k, "2d", 4, None) for k in ("gpt2", "roberta", "albert", "t5", "bart", "opt", "blenderbot", "vit", "bert_cls", "bert_qa")]
ND_CASES += [("bart", "2.5d", 8, 2), ("t5", "3d", 8, None), ("vit", "3d", 8, None), ("bert_cls", "3d", 8, None)]


@pytest.mark.parametrize("kind,mode,world,depth", ND_CASES, ids=[f"{c[0]}-{c[1]}" for c in ND_CASES])
def test_hf_model_tensor_parallel_nd(kind, mode, world, depth):
    run_dist(_nd_worker, world, kind, mode, depth, timeout=600)


def _pp_worker(rank, world, kind):
    """Stock Hugging Face model, no ``pipeline_units()``: the module tree is cut into two stages."""
    import oslo_b200
    from oslo_b200 import ParallelContext
    from oslo_b200.parallel import PipelineParallel

    pc = ParallelContext.from_torch(pipeline_parallel_size=world, backend="gloo", seed=0)
    ref = _build(kind).train()
    model = _build(kind).train()
    wrapped = PipelineParallel(model, pc, num_micro_batches=2)
    oslo_b200.ready(wrapped, pc)
    assert wrapped._tree is not None
    released = [n for n, p in model.named_parameters() if getattr(p, "oslo_pipeline_released", False)]
    assert released, "every stage still holds the whole model"
    ids = torch.randint(0, 100, (4, 12), generator=torch.Generator().manual_seed(1))
    ref_loss = sum(ref(input_ids=c, labels=c).loss for c in ids.chunk(2)) / 2
    ref_loss.backward()
    total = 0.0
    for _, out in wrapped(input_ids=ids, labels=ids):
        out.loss.backward()
        if wrapped.stage == world - 1:
            total += out.loss.item()
    if wrapped.stage == world - 1:
        assert abs(total - ref_loss.item()) < 1e-4, (total, ref_loss.item())
    ref_grads = dict(ref.named_parameters())
    checked = 0
    for n, p in model.named_parameters():
        if getattr(p, "oslo_pipeline_released", False) or p.grad is None:
            continue
        g = ref_grads[n].grad
        assert torch.allclose(p.grad, g, rtol=1e-3, atol=1e-5), (n, (p.grad - g).abs().max().item())
        checked += 1
    assert checked > 5
    pc.destroy()


@pytest.mark.parametrize("kind", ["gpt2", "gpt_neox", "bert", "llama", "opt"])  # opt registers its closing norm BEFORE the blocks
def test_hf_model_pipeline_parallel_from_module_tree(kind):
    run_dist(_pp_worker, 2, kind, timeout=600)


def _vp_loss_worker(rank, world, kind):
    """Stock Hugging Face causal LM under 1-D TensorParallel with the vocab-parallel loss: the head's logits stay
    sharded over the vocabulary, loss and gradients equal the unsharded model's."""
    import oslo_b200
    from oslo_b200 import ParallelContext
    from oslo_b200.parallel import TensorParallel
    from oslo_b200.parallel.tensor_parallel._sharding import merge

    pc = ParallelContext.from_torch(tensor_parallel_size=world, backend="gloo", seed=0)
    ref = _build(kind).train()
    model = _build(kind).train()
    wrapped = TensorParallel(model, pc, vocab_parallel_loss=True)
    oslo_b200.ready(wrapped, pc)
    ids = torch.randint(0, 100, (2, 12), generator=torch.Generator().manual_seed(1))
    want = ref(input_ids=ids, labels=ids)
    want.loss.backward()
    got = wrapped(input_ids=ids, labels=ids)
    got.loss.backward()
    assert got.logits.shape[-1] == want.logits.shape[-1] // world  # a vocabulary slice, never the gathered logits
    assert torch.allclose(got.loss, want.loss, rtol=1e-5, atol=1e-6), (got.loss.item(), want.loss.item())
    ref_grads = {k: p.grad for k, p in ref.named_parameters()}
    checked = 0
    for k, p in model.named_parameters():
        g = merge(p.grad, p.oslo_shard, pc) if hasattr(p, "oslo_shard") else p.grad
        full = ref_grads[k]
        g = g[: full.shape[0]] if g.shape != full.shape else g
        assert torch.allclose(g, full, rtol=1e-3, atol=1e-5), (k, (g - full).abs().max().item())
        checked += 1
    assert checked > 8
    pc.destroy()


@pytest.mark.parametrize("kind", ["gpt2", "gpt_neox", "llama"])
def test_hf_causal_lm_with_vocab_parallel_loss(kind):
    run_dist(_vp_loss_worker, 2, kind, timeout=600)


@pytest.mark.parametrize("kind", ["gpt_neox", "llama", "bert"])
def test_kernel_fusion_surgery_keeps_hf_outputs(kind):
    """``fuse_all``: norms, linears and attention of a stock Hugging Face model go through this library's ops
    (their torch paths on CPU) without changing the outputs."""
    from oslo_b200.transformers.kernel_fusion_utils import fuse_all

    import oslo_b200.nn as onn

    ref = _build(kind)
    model = fuse_all(_build(kind))
    assert model.config._attn_implementation == "oslo_b200"
    assert any(isinstance(m, onn.Linear) for m in model.modules())
    assert not any(type(m) is torch.nn.LayerNorm for m in model.modules())
    ids = torch.randint(0, 100, (2, 12), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = ref(input_ids=ids).logits
        got = model(input_ids=ids).logits
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-5), (got - want).abs().max()


def _ep_worker(rank, world, kind):
    """Stock Hugging Face models under expert parallelism: the mapped feed-forward linears (and only those: an attention
    output projection with the same name suffix stays dense) become router + experts, the experts are spread over the
    group, forward / backward run and every expert parameter receives a gradient."""
    import oslo_b200
    from oslo_b200 import ParallelContext
    from oslo_b200.parallel import ExpertParallel
    from oslo_b200.parallel.expert_parallel.layers import ExpertParallelBehindBlock, ExpertParallelFrontBlock

    pc = ParallelContext.from_torch(expert_parallel_size=world, backend="gloo", seed=0)
    model = _build(kind).train()
    encoder_only = kind in ("bert", "roberta", "albert", "electra", "distilbert", "vit")
    both = kind in ("t5", "bart", "blenderbot")
    kw = dict(top_k=2, capacity_factor_train=4.0, aux_loss_coef=0.01)
    if encoder_only or both:
        kw["num_enc_experts"] = 4
    if not encoder_only:
        kw["num_dec_experts"] = 4
    wrapped = ExpertParallel(model, pc, **kw)
    oslo_b200.ready(wrapped, pc)
    fronts = [n for n, m in model.named_modules() if isinstance(m, ExpertParallelFrontBlock)]
    behinds = [n for n, m in model.named_modules() if isinstance(m, ExpertParallelBehindBlock)]
    assert len(fronts) == len(behinds) >= 2 and not any("attention" in n or "attn" in n.split(".")[-2] for n in behinds), (fronts, behinds)
    feed = _inputs(kind)
    if kind == "vit":
        feed["labels"] = torch.tensor([1, 2])
    else:
        feed["labels"] = feed.pop("decoder_input_ids", feed["input_ids"]).clone() if both else feed["input_ids"].clone()
    out = wrapped(**feed)
    assert torch.isfinite(out.loss)
    out.loss.backward()
    experts = [(n, p) for n, p in model.named_parameters() if getattr(p, "oslo_expert_param", False)]
    assert experts and all(p.shape[0] == 4 // world and p.grad is not None and torch.isfinite(p.grad).all() for _, p in experts)
    pc.destroy()


@pytest.mark.parametrize("kind", ["bert", "t5", "bart", "gptj", "vit", "distilbert"])
def test_hf_model_expert_parallel(kind):
    run_dist(_ep_worker, 2, kind, timeout=600)


def _deparallel_worker(rank, world, kind):
    """Shard a stock model over a 2-D grid and merge it back in memory: same state dict, same outputs, and the layers that
    were swapped for parallel ones are the library's own classes again (scaled / learned-position embeddings, RMS norms)."""
    import oslo_b200
    from oslo_b200 import ParallelContext, ParallelMode
    from oslo_b200.parallel import TensorParallel

    pc = ParallelContext.from_torch(tensor_parallel_size=world, tensor_parallel_mode=ParallelMode.TENSOR_2D, backend="gloo", seed=0)
    ref, model = _build(kind), _build(kind)
    classes = {n: type(m).__name__ for n, m in ref.named_modules(remove_duplicate=False) if isinstance(m, torch.nn.Embedding)}
    wrapped = TensorParallel(model, pc)
    oslo_b200.ready(wrapped, pc)
    wrapped.deparallelize()
    state, ref_state = model.state_dict(), ref.state_dict()
    assert set(state) == set(ref_state) and all(torch.equal(state[k], v) for k, v in ref_state.items())
    # (tables that were separate modules around one tied weight come back as one module under all their names)
    after = {n: type(m).__name__ for n, m in model.named_modules(remove_duplicate=False) if isinstance(m, torch.nn.Embedding)}
    assert after == classes, (after, classes)
    feed = {k: torch.cat([v, v]) for k, v in _inputs(kind).items()}
    with torch.no_grad():
        assert torch.allclose(model(**feed).logits, ref(**feed).logits, rtol=1e-4, atol=1e-5)
    pc.destroy()


@pytest.mark.parametrize("kind", ["bart", "t5", "opt"])
def test_hf_model_deparallelize_after_2d(kind):
    run_dist(_deparallel_worker, 4, kind, timeout=600)


def _tp_pp_worker(rank, world, kind):
    """Stock model, 2-D tensor parallel inside each of two pipeline stages cut from the module tree: the stage that does
    not own the embeddings stands in for them with placeholders of the sharded width."""
    import oslo_b200
    from oslo_b200 import ParallelContext, ParallelMode
    from oslo_b200.parallel import PipelineParallel, TensorParallel

    pc = ParallelContext.from_torch(tensor_parallel_size=4, pipeline_parallel_size=2, tensor_parallel_mode=ParallelMode.TENSOR_2D,
                                    backend="gloo", seed=0)
    ref, model = _build(kind).train(), _build(kind).train()
    TensorParallel(model, pc)
    wrapped = PipelineParallel(model, pc, num_micro_batches=2)
    oslo_b200.ready(wrapped, pc)
    ids = torch.randint(0, 100, (8, 12), generator=torch.Generator().manual_seed(1))
    ref_loss = sum(ref(input_ids=c, labels=c).loss for c in ids.chunk(2)) / 2
    total = 0.0
    for _, out in wrapped(input_ids=ids, labels=ids):
        if out.loss is not None:
            out.loss.backward()
            if wrapped.stage == 1:
                total += out.loss.item()
    if wrapped.stage == 1:
        assert abs(total - ref_loss.item()) < 1e-4, (total, ref_loss.item())
    pc.destroy()


def test_hf_model_2d_tensor_parallel_inside_pipeline_stages():
    run_dist(_tp_pp_worker, 8, "gpt2", timeout=900)


def _vp_loss_other_worker(rank, world, kind):
    """``vocab_parallel_loss=True`` beyond causal models: masked-LM labels are used as they are, encoder-decoder models
    get the decoder inputs the library would have derived from the labels, and BART's per-token logits bias is added
    slice by slice; the loss equals the unsharded model's and gradients flow."""
    import oslo_b200
    from oslo_b200 import ParallelContext
    from oslo_b200.parallel import TensorParallel

    pc = ParallelContext.from_torch(tensor_parallel_size=world, backend="gloo", seed=0)
    ref, model = _build(kind), _build(kind)
    if kind == "bart":
        with torch.no_grad():
            bias = torch.randn(1, 100, generator=torch.Generator().manual_seed(3))
            ref.final_logits_bias.copy_(bias)
            model.final_logits_bias.copy_(bias)
    wrapped = TensorParallel(model, pc, vocab_parallel_loss=True)
    oslo_b200.ready(wrapped, pc)
    feed = _inputs(kind)
    labels = feed.pop("decoder_input_ids", feed["input_ids"]).clone()
    labels[0, :2] = -100
    want = ref(**feed, labels=labels).loss
    out = wrapped(**feed, labels=labels)
    assert torch.allclose(out.loss, want, atol=1e-5), (kind, float(out.loss), float(want))
    assert out.logits.shape[-1] == 100 // world  # the head's output stays sharded
    out.loss.backward()
    pc.destroy()


@pytest.mark.parametrize("kind", ["bert", "t5", "bart"])
def test_hf_vocab_parallel_loss_masked_and_encoder_decoder(kind):
    run_dist(_vp_loss_other_worker, 2, kind, timeout=600)


def _reload_worker(rank, world, kind, two_d, tmp):
    """Per-rank shards written by ``save_pretrained`` load back into a freshly sharded copy with other weights
    (``from_parallelized``), including tables that several modules share."""
    import oslo_b200
    from oslo_b200 import ParallelContext, ParallelMode
    from oslo_b200.parallel import TensorParallel

    pc = ParallelContext.from_torch(tensor_parallel_size=world, backend="gloo", seed=0,
                                    tensor_parallel_mode=ParallelMode.TENSOR_2D if two_d else ParallelMode.TENSOR_1D)
    ref, first = _build(kind), _build(kind)
    saved = TensorParallel(first, pc)
    oslo_b200.ready(saved, pc)
    saved.save_pretrained(tmp)
    torch.distributed.barrier()
    other = _build(kind)
    with torch.no_grad():
        for p in other.parameters():
            p.mul_(0.5)
    loaded = TensorParallel(other, pc)
    oslo_b200.ready(loaded, pc)
    loaded.from_parallelized(tmp)
    feed = {k: torch.cat([v, v]) for k, v in _inputs(kind).items()}
    with torch.no_grad():
        assert torch.allclose(loaded(**feed).logits, ref(**feed).logits, rtol=1e-4, atol=1e-5)
    pc.destroy()


@pytest.mark.parametrize("kind,world,two_d", [("bart", 2, False), ("t5", 4, True)])
def test_hf_model_sharded_checkpoint_reload(kind, world, two_d):
    with tempfile.TemporaryDirectory() as tmp:
        run_dist(_reload_worker, world, kind, two_d, tmp, timeout=600)
