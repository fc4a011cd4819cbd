"""2D / 2.5D / 3D tensor parallelism on CPU / gloo: loss and merged gradients equal the unsharded model."""
import os
import tempfile

import pytest
import torch

from dist_utils import run_dist


def _neox(seed=0):
    from oslo_b200.models.config import GPTNeoXConfig
    from oslo_b200.models.gpt_neox import GPTNeoXForCausalLM

    torch.manual_seed(seed)
    cfg = GPTNeoXConfig(vocab_size=250, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                        intermediate_size=128, max_position_embeddings=32)
    return GPTNeoXForCausalLM(cfg)


def _worker(rank, world, mode_name, depth, tmp):
    import oslo_b200
    from oslo_b200 import ParallelContext, ParallelMode
    from oslo_b200.parallel import TensorParallel
    from oslo_b200.parallel.tensor_parallel._sharding import merge

    pc = ParallelContext.from_torch(tensor_parallel_size=world, tensor_parallel_mode=mode_name,
                                    tensor_parallel_depth=depth, backend="gloo", seed=0)
    ref = _neox()
    model = _neox()
    ref_state = {k: v.clone() for k, v in ref.state_dict().items()}
    wrapped = TensorParallel(model, pc)
    oslo_b200.ready(wrapped, pc)
    torch.manual_seed(1)
    ids = torch.randint(0, 250, (8, 16))
    out_ref = ref(input_ids=ids, labels=ids)
    out_ref.loss.backward()
    out = wrapped(input_ids=ids, labels=ids)
    out.loss.backward()
    assert torch.allclose(out.loss, out_ref.loss, rtol=1e-5, atol=1e-6), (out.loss.item(), out_ref.loss.item())
    ref_grads = {k: p.grad for k, p in ref.named_parameters()}
    checked = 0
    for k, p in model.named_parameters():
        g = p.grad
        full = ref_grads[k]
        if hasattr(p, "oslo_shard"):
            spec = p.oslo_shard
            saved = spec.full_shape
            spec.full_shape = None  # keep vocabulary padding for the comparison below
            g = merge(g, spec, pc)
            spec.full_shape = saved
            g = g[tuple(slice(0, n) for n in full.shape)]
        assert torch.allclose(g, full, rtol=2e-4, atol=2e-6), (mode_name, k, (g - full).abs().max().item())
        checked += 1
    assert checked > 10
    wrapped.save_pretrained(tmp, merge_checkpoints=True)
    if rank == 0:
        merged = torch.load(os.path.join(tmp, "pytorch_model.bin"))
        for k, v in ref_state.items():
            assert torch.equal(merged[k], v), k
    pc.destroy()


@pytest.mark.parametrize("mode,world,depth", [("2d", 4, None), ("2.5d", 8, 2), ("3d", 8, None)])
def test_neox_nd_matches_unsharded(mode, world, depth):
    with tempfile.TemporaryDirectory() as tmp:
        run_dist(_worker, world, mode, depth, tmp, timeout=600)
