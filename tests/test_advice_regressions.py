"""Regression tests on CPU / gloo for state handling around wrappers:

* ZeRO: the fp32 master shards follow weights loaded after wrapping, and a saved optimizer state resumes identically;
* ZeRO with overlapped reduction and gradient accumulation (``no_sync``), and the error without it;
* ``TensorParallel.deparallelize`` restores the per-module arguments it divided, so the model runs again unsharded;
* ``save_pretrained(merge_checkpoints=True)`` and the sharded round trip with tensor x pipeline parallelism.
"""
import os
import tempfile

import pytest
import torch
import torch.nn as nn

from dist_utils import run_dist


def _mlp(seed=0):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Linear(16, 32), nn.GELU(), nn.Linear(32, 32), nn.LayerNorm(32), nn.Linear(32, 4))


def _data(step, n=8):
    g = torch.Generator().manual_seed(100 + step)
    return torch.randn(n, 16, generator=g), torch.randn(n, 4, generator=g)


def _train(model, opt, rank, world, steps, first=0):
    for s in range(first, first + steps):
        x, y = _data(s)
        xs, ys = x.chunk(world)[rank], y.chunk(world)[rank]
        opt.zero_grad()
        opt.backward(((model(xs) - ys) ** 2).mean())
        opt.step()


def _zero_resume_worker(rank, world, stage, with_state):
    from oslo_b200 import ParallelContext
    from oslo_b200.parallel import ZeroRedundancyOptimizer

    pc = ParallelContext.from_torch(data_parallel_size=world, backend="gloo", seed=0)

    def make(model):
        return ZeroRedundancyOptimizer(torch.optim.AdamW(model.parameters(), lr=1e-2), parallel_context=pc,
                                       partition_grad=stage == 2, reduce_bucket_size=600)

    # uninterrupted run: 4 steps
    full = _mlp()
    _train(full, make(full), rank, world, 4)
    # interrupted run: 2 steps, "checkpoint", new process state, 2 more steps
    a = _mlp()
    opt_a = make(a)
    _train(a, opt_a, rank, world, 2)
    weights = {k: v.clone() for k, v in a.state_dict().items()}
    opt_sd = opt_a.state_dict()
    b = _mlp(seed=7)  # different initial weights: the optimizer is built BEFORE the checkpoint is loaded
    opt_b = make(b)
    b.load_state_dict(weights)
    if with_state:
        opt_b.load_state_dict(opt_sd)
        _train(b, opt_b, rank, world, 2, first=2)
        for p, r in zip(b.parameters(), full.parameters()):
            assert torch.allclose(p, r, rtol=1e-5, atol=1e-6), (p - r).abs().max()
    else:
        opt_b.resync_master()
        _train(b, opt_b, rank, world, 1, first=2)
        # one AdamW step moves a weight by about lr; stale masters would throw the weights back to seed-7 values
        for p, w in zip(b.parameters(), weights.values()):
            assert (p - w).abs().max() < 0.05, (p - w).abs().max()
    pc.destroy()


@pytest.mark.parametrize("stage,with_state", [(1, True), (2, True), (1, False)])
def test_zero_resume_keeps_master_weights(stage, with_state):
    run_dist(_zero_resume_worker, 2, stage, with_state)


def _zero_accum_worker(rank, world, use_no_sync):
    from oslo_b200 import ParallelContext
    from oslo_b200.parallel import ZeroRedundancyOptimizer

    pc = ParallelContext.from_torch(data_parallel_size=world, backend="gloo", seed=0)
    model = _mlp()
    opt = ZeroRedundancyOptimizer(torch.optim.AdamW(model.parameters(), lr=1e-2), parallel_context=pc, partition_grad=True,
                                  overlap_communication=True, reduce_bucket_size=600)
    ref = _mlp()
    ref_opt = torch.optim.AdamW(ref.parameters(), lr=1e-2)
    for s in range(3):
        ref_opt.zero_grad()
        opt.zero_grad()
        for micro in range(2):
            x, y = _data(2 * s + micro)
            (((ref(x) - y) ** 2).mean() / 2).backward()
            xs, ys = x.chunk(world)[rank], y.chunk(world)[rank]
            loss = ((model(xs) - ys) ** 2).mean() / 2
            if micro == 0 and use_no_sync:
                with opt.no_sync():
                    opt.backward(loss)
            elif micro == 0:
                opt.backward(loss)
            else:
                if use_no_sync:
                    opt.backward(loss)
                else:
                    with pytest.raises(RuntimeError, match="no_sync"):
                        opt.backward(loss)
                    pc.destroy()
                    return
        ref_opt.step()
        opt.step()
    for p, r in zip(model.parameters(), ref.parameters()):
        assert torch.allclose(p, r, rtol=1e-5, atol=1e-6), (p - r).abs().max()
    pc.destroy()


@pytest.mark.parametrize("use_no_sync", [True, False])
def test_zero_overlap_with_gradient_accumulation(use_no_sync):
    run_dist(_zero_accum_worker, 2, use_no_sync)


def _gpt2_hf():
    from transformers import GPT2Config, GPT2LMHeadModel

    torch.manual_seed(0)
    return GPT2LMHeadModel(GPT2Config(vocab_size=100, n_positions=32, n_embd=32, n_layer=2, n_head=4, resid_pdrop=0.0,
                                      embd_pdrop=0.0, attn_pdrop=0.0)).eval()


def _deparallelize_worker(rank, world, mode_name):
    import oslo_b200
    from oslo_b200 import ParallelContext, ParallelMode
    from oslo_b200.parallel import TensorParallel

    mode = getattr(ParallelMode, mode_name)
    pc = ParallelContext.from_torch(tensor_parallel_size=world, tensor_parallel_mode=mode, backend="gloo", seed=0)
    ref, model = _gpt2_hf(), _gpt2_hf()
    wrapped = TensorParallel(model, pc)
    oslo_b200.ready(wrapped, pc)
    ids = torch.randint(0, 100, (4, 12), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = ref(input_ids=ids).logits
        assert torch.allclose(wrapped(input_ids=ids).logits[..., :100], want, rtol=1e-4, atol=1e-5)
    wrapped.deparallelize()
    with torch.no_grad():
        got = model(input_ids=ids).logits  # the bare module, unsharded again
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-5), (got - want).abs().max()
    for (k, v), (_, r) in zip(sorted(model.state_dict().items()), sorted(ref.state_dict().items())):
        assert v.shape == r.shape, k
    pc.destroy()


@pytest.mark.parametrize("world,mode", [(2, "TENSOR_1D"), (4, "TENSOR_2D")])
def test_forward_after_deparallelize(world, mode):
    run_dist(_deparallelize_worker, world, mode, timeout=600)


def _llama(seed=0):
    from oslo_b200.models import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(seed)
    return LlamaForCausalLM(LlamaConfig(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=4,
                                        num_attention_heads=4, max_position_embeddings=32))


def _tp_pp_ckpt_worker(rank, world, mode_name, tp, tmp):
    import oslo_b200
    from oslo_b200 import ParallelContext, ParallelMode
    from oslo_b200.parallel import PipelineParallel, TensorParallel

    pc = ParallelContext.from_torch(tensor_parallel_size=tp, pipeline_parallel_size=2,
                                    tensor_parallel_mode=getattr(ParallelMode, mode_name), backend="gloo", seed=0)
    ref = _llama()
    full = {k: v.clone() for k, v in ref.state_dict().items()}

    def build(seed):
        m = _llama(seed)
        TensorParallel(m, pc)
        w = PipelineParallel(m, pc, num_micro_batches=2)
        oslo_b200.ready(w, pc)
        return m, w

    model, wrapped = build(0)
    merged_dir, shard_dir = os.path.join(tmp, "merged"), os.path.join(tmp, "shards")
    wrapped.save_pretrained(merged_dir, merge_checkpoints=True)
    if rank == 0:
        merged = torch.load(os.path.join(merged_dir, "pytorch_model.bin"))
        assert set(merged) == set(full), set(full) ^ set(merged)
        for k, v in full.items():
            assert merged[k].shape == v.shape, (k, merged[k].shape, v.shape)
            assert torch.equal(merged[k], v), k
    # sharded round trip into a differently initialised model
    wrapped.save_pretrained(shard_dir)
    other, other_wrapped = build(5)
    other_wrapped.from_parallelized(shard_dir)
    for (k, a), (_, b) in zip(model.state_dict().items(), other.state_dict().items()):
        assert torch.equal(a, b), k
    pc.destroy()


@pytest.mark.parametrize("mode,tp,world", [("TENSOR_1D", 2, 4), ("TENSOR_2D", 4, 8)])
def test_tensor_x_pipeline_checkpoints(mode, tp, world):
    with tempfile.TemporaryDirectory() as tmp:
        run_dist(_tp_pp_ckpt_worker, world, mode, tp, tmp, timeout=900)


def test_fused_reduce_scatter_policy_by_group_size(monkeypatch):
    """The row-parallel side leaves the fused kernel above FUSED_RS_MAX_RANKS ranks; the all-gather side never does."""
    import torch

    from oslo_b200.ops import fused_collectives as fc
    from oslo_b200.parallel.tensor_parallel import _ops_1d

    class _WS:
        def __init__(self, tp):
            self.tp = tp

        def ag_ok(self, x, w):
            return True

        def rs_ok(self, x, w, along_n=False):
            return True

    class _RT:
        def __init__(self, tp):
            self.ws = _WS(tp)

    class _FakeCuda(torch.Tensor):
        is_cuda = True

    x = torch.zeros(4, 4).as_subclass(_FakeCuda)
    assert _ops_1d.FUSED_RS_MAX_RANKS == 8  # default: fused at every size of one node (the configuration measured end to end)
    monkeypatch.setattr(_ops_1d, "FUSED_RS_MAX_RANKS", 4)
    for tp, want_rs in ((2, True), (4, True), (8, False)):
        monkeypatch.setattr(fc, "_runtime", _RT(tp))
        assert _ops_1d._use_fused(x, x, "rs") is want_rs, tp
        assert _ops_1d._use_fused(x, x, "ag") is True
    monkeypatch.setattr(_ops_1d, "FUSED_RS_MAX_RANKS", 8)
    assert _ops_1d._use_fused(x, x, "rs") is True
    monkeypatch.setattr(fc, "_runtime", None)
    assert _ops_1d._use_fused(x, x, "rs") is False
