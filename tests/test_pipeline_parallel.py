"""Pipeline parallelism (1F1B over gloo p2p): loss and gradients equal the unsplit model; partitioner properties."""
import pytest
import torch

from dist_utils import run_dist


def test_partitioner_balances_contiguously():
    import torch.nn as nn

    from oslo_b200.parallel.pipeline_parallel import ModelPartitioner, PipeUnit

    sizes = [10, 1, 1, 1, 1, 10, 2, 2]
    units = [PipeUnit(str(i), [nn.Linear(n, 100, bias=False)], lambda s: s) for i, n in enumerate(sizes)]
    part = ModelPartitioner(units, 3).partition()
    assert [list(r) for r in part] == [[0], [1, 2, 3, 4], [5, 6, 7]] or max(
        sum(sizes[i] for i in r) for r in part) <= 14
    flat = [i for r in part for i in r]
    assert flat == list(range(len(sizes)))  # contiguous, complete, ordered


def _gpt2(seed=0):
    from oslo_b200.models.config import GPT2Config
    from oslo_b200.models.gpt2 import GPT2LMHeadModel

    torch.manual_seed(seed)
    cfg = GPT2Config(vocab_size=128, n_positions=32, n_embd=32, n_layer=4, n_head=4, resid_pdrop=0.0, embd_pdrop=0.0,
                     attn_pdrop=0.0)
    return GPT2LMHeadModel(cfg)


def _worker(rank, world, micro):
    import oslo_b200
    from oslo_b200 import ParallelContext
    from oslo_b200.parallel import PipelineParallel

    pc = ParallelContext.from_torch(pipeline_parallel_size=world, backend="gloo", seed=0)
    ref = _gpt2()
    model = _gpt2()
    wrapped = PipelineParallel(model, pc, num_micro_batches=micro)
    oslo_b200.ready(wrapped, pc)
    torch.manual_seed(3)
    ids = torch.randint(0, 128, (4, 16))
    # reference: mean of per-micro-batch losses = what the pipeline accumulates
    ref_loss = 0.0
    for chunk in ids.chunk(micro):
        o = ref(input_ids=chunk, labels=chunk)
        (o.loss / micro).backward()
        ref_loss += o.loss.item() / micro
    total = 0.0
    for ind, out in wrapped(input_ids=ids, labels=ids):
        out.loss.backward()
        if wrapped.stage == world - 1:
            total += out.loss.item()
    if wrapped.stage == world - 1:
        assert abs(total - ref_loss) < 1e-5, (total, ref_loss)
    ref_params = dict(ref.named_parameters())
    checked = 0
    for name, p in model.named_parameters():
        if getattr(p, "oslo_pipeline_released", False):
            assert p.numel() == 0
            continue
        assert p.grad is not None, name
        assert torch.allclose(p.grad, ref_params[name].grad, rtol=1e-4, atol=1e-6), (name, (p.grad - ref_params[name].grad).abs().max())
        checked += 1
    assert checked > 3
    pc.destroy()


@pytest.mark.parametrize("world,micro", [(2, 2), (2, 4), (4, 4)])
def test_pipeline_matches_unsplit_model(world, micro):
    run_dist(_worker, world, micro)


def _llama(seed=0):
    from oslo_b200.models import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(seed)
    return LlamaForCausalLM(LlamaConfig(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=4,
                                        num_attention_heads=4, max_position_embeddings=32))


def _pp_tp2d_worker(rank, world):
    import oslo_b200
    from oslo_b200 import ParallelContext, ParallelMode
    from oslo_b200.parallel import PipelineParallel, TensorParallel

    pc = ParallelContext.from_torch(tensor_parallel_size=4, pipeline_parallel_size=2, tensor_parallel_mode=ParallelMode.TENSOR_2D,
                                    backend="gloo", seed=0)
    ref = _llama()
    model = _llama()
    TensorParallel(model, pc)
    wrapped = PipelineParallel(model, pc, num_micro_batches=2)
    oslo_b200.ready(wrapped, pc)
    torch.manual_seed(3)
    ids = torch.randint(0, 128, (8, 16))
    ref_loss = sum(ref(input_ids=c, labels=c).loss.item() for c in ids.chunk(2)) / 2
    total = 0.0
    for _, out in wrapped(input_ids=ids, labels=ids):
        out.loss.backward()
        if wrapped.stage == 1:
            total += out.loss.item()
    if wrapped.stage == 1:
        assert abs(total - ref_loss) < 1e-4, (total, ref_loss)
    pc.destroy()


def test_pipeline_with_2d_tensor_parallel():
    run_dist(_pp_tp2d_worker, 8, timeout=900)


def _seq2seq(kind):
    from oslo_b200 import models

    torch.manual_seed(0)
    if kind == "t5":
        return models.T5ForConditionalGeneration(models.T5Config(vocab_size=96, d_model=32, d_kv=8, d_ff=64, num_layers=3,
                                                                 num_decoder_layers=3, num_heads=4, dropout_rate=0.0))
    return models.BartForConditionalGeneration(models.BartConfig(
        vocab_size=96, d_model=32, encoder_layers=3, decoder_layers=3, encoder_attention_heads=4, decoder_attention_heads=4,
        encoder_ffn_dim=64, decoder_ffn_dim=64, max_position_embeddings=32, dropout=0.0, attention_dropout=0.0,
        activation_dropout=0.0))


def _seq2seq_worker(rank, world, kind):
    """Encoder-decoder models through the pipeline: the encoder output and the decoder state travel as one activation, the
    loss and every gradient (including parameters kept on several stages: the shared embedding, T5's relative-position
    tables) equal those of the unsplit model."""
    import oslo_b200
    from oslo_b200 import ParallelContext
    from oslo_b200.parallel import PipelineParallel

    pc = ParallelContext.from_torch(pipeline_parallel_size=world, backend="gloo", seed=0)
    ref, model = _seq2seq(kind), _seq2seq(kind)
    wrapped = PipelineParallel(model, pc, num_micro_batches=2)
    oslo_b200.ready(wrapped, pc)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(3, 96, (4, 11), generator=g)
    labels = torch.randint(3, 96, (4, 7), generator=g)
    mask = torch.ones_like(ids)
    mask[1, 8:] = 0
    ref_loss = sum(ref(input_ids=i, attention_mask=m, labels=l).loss for i, m, l in zip(ids.chunk(2), mask.chunk(2), labels.chunk(2))) / 2
    ref_loss.backward()
    total = 0.0
    for _, out in wrapped(input_ids=ids, attention_mask=mask, labels=labels):
        out.loss.backward()
        if wrapped.stage == world - 1:
            total += out.loss.item()
    if wrapped.stage == world - 1:
        assert abs(total - ref_loss.item()) < 1e-4, (total, ref_loss.item())
    ref_grads = {n: p.grad for n, p in ref.named_parameters()}
    checked = 0
    for n, p in model.named_parameters():
        if getattr(p, "oslo_pipeline_released", False) or p.grad is None:
            continue
        assert torch.allclose(p.grad, ref_grads[n], rtol=1e-3, atol=1e-5), (kind, n, (p.grad - ref_grads[n]).abs().max().item())
        checked += 1
    assert checked > 5
    released = [n for n, p in model.named_parameters() if getattr(p, "oslo_pipeline_released", False)]
    assert released, "every stage still holds the whole model"
    pc.destroy()


@pytest.mark.parametrize("kind,world", [("bart", 2), ("t5", 2), ("t5", 4)])
def test_pipeline_encoder_decoder_models(kind, world):
    run_dist(_seq2seq_worker, world, kind)
