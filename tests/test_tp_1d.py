"""1-D tensor parallelism on CPU / gloo: loss and gradients equal the unsharded model, with and without
sequence parallelism; merged checkpoint equals the original weights."""
import os
import tempfile

import pytest
import torch

from dist_utils import run_dist


def _neox(seed=0):
    from oslo_b200.models.config import GPTNeoXConfig
    from oslo_b200.models.gpt_neox import GPTNeoXForCausalLM

    torch.manual_seed(seed)
    cfg = GPTNeoXConfig(vocab_size=509, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                        intermediate_size=128, max_position_embeddings=32)
    model = GPTNeoXForCausalLM(cfg)
    # non-trivial LayerNorm parameters and biases, so that folding them into the next weights is really exercised
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "layernorm" in n or "layer_norm" in n or n.endswith(".bias"):
                p.add_(torch.randn_like(p) * 0.3)
    return model


def _worker(rank, world, sp, tmp):
    import oslo_b200
    from oslo_b200 import ParallelContext, ParallelMode
    from oslo_b200.parallel import TensorParallel
    from oslo_b200.parallel.tensor_parallel._sharding import merge

    pc = ParallelContext.from_torch(tensor_parallel_size=world, tensor_parallel_mode=ParallelMode.TENSOR_1D,
                                    backend="gloo", seed=0)
    ref = _neox()
    model = _neox()
    ref_state = {k: v.clone() for k, v in ref.state_dict().items()}
    wrapped = TensorParallel(model, pc, sequence_parallel=sp)
    oslo_b200.ready(wrapped, pc)
    torch.manual_seed(1)
    ids = torch.randint(0, 509, (world * 2, 16))
    out_ref = ref(input_ids=ids, labels=ids)
    out_ref.loss.backward()
    out = wrapped(input_ids=ids, labels=ids)
    out.loss.backward()
    assert torch.allclose(out.loss, out_ref.loss, rtol=1e-5, atol=1e-6), (out.loss.item(), out_ref.loss.item())
    ref_grads = {k: p.grad for k, p in ref.named_parameters()}
    checked = 0
    for k, p in model.named_parameters():
        g = p.grad
        if hasattr(p, "oslo_shard"):
            g = merge(g, p.oslo_shard, pc)
            full = ref_grads[k]
            if g.shape != full.shape:  # vocabulary padding
                full = torch.nn.functional.pad(full, (0, 0, 0, g.shape[0] - full.shape[0])) if g.dim() == 2 else full
            g = g[: full.shape[0]]
        else:
            full = ref_grads[k]
        assert torch.allclose(g, full, rtol=1e-4, atol=1e-6), (k, (g - full).abs().max().item())
        checked += 1
    assert checked > 10
    wrapped.save_pretrained(tmp, merge_checkpoints=True)
    wrapped.save_pretrained(tmp)
    if rank == 0:
        merged = torch.load(os.path.join(tmp, "pytorch_model.bin"))
        for k, v in ref_state.items():
            assert torch.equal(merged[k], v), k
    assert os.path.isfile(os.path.join(tmp, f"pytorch_model_tp_{rank}_pp_0_ep_0.bin"))
    # reload the per-rank shards into a freshly sharded model
    model2 = _neox(seed=5)
    w2 = TensorParallel(model2, pc, sequence_parallel=sp)
    oslo_b200.ready(w2, pc)
    w2.from_parallelized(tmp)
    out2 = w2(input_ids=ids, labels=ids)
    assert torch.allclose(out2.loss, out_ref.loss, rtol=1e-5, atol=1e-6)
    pc.destroy()


@pytest.mark.parametrize("sp", [False, True])
def test_neox_tp2_matches_unsharded(sp):
    with tempfile.TemporaryDirectory() as tmp:
        run_dist(_worker, 2, sp, tmp)
