"""Mixture of experts: routing ops against the dense GShard formulation, and EP=2 against EP=1 (CPU / gloo)."""
import math

import pytest
import torch
import torch.nn.functional as F

from dist_utils import run_dist


def test_positions_dispatch_combine_match_dense_formulation():
    from oslo_b200.ops import moe

    torch.manual_seed(0)
    S, E, K, H, C = 37, 4, 2, 16, 12
    idx = torch.stack([torch.randint(0, E, (S,)), torch.randint(0, E, (S,))], 1)
    pos, counts = moe.positions(idx.to(torch.int32), E)
    # dense reference: cumsum over one-hot masks, second choices offset by the first-choice counts
    m1, m2 = F.one_hot(idx[:, 0], E), F.one_hot(idx[:, 1], E)
    l1 = (torch.cumsum(m1, 0) - 1) * m1
    l2 = (torch.cumsum(m2, 0) - 1 + m1.sum(0, keepdim=True)) * m2
    assert torch.equal(pos[:, 0].long(), l1.sum(1)) and torch.equal(pos[:, 1].long(), l2.sum(1))
    assert torch.equal(counts.long(), (m1 + m2).sum(0))
    kept = pos < C
    slot = torch.where(kept, idx.to(torch.int32) * C + pos, torch.full_like(pos, -1))
    x = torch.randn(S, H, requires_grad=True)
    w = torch.rand(S, K, requires_grad=True)
    buf = moe.dispatch(x, slot, E * C)
    y = moe.combine(buf * 2.0, w, slot)
    # einsum formulation
    sec = torch.zeros(S, E, C)
    for s in range(S):
        for k in range(K):
            if slot[s, k] >= 0:
                sec[s, slot[s, k] // C, slot[s, k] % C] = 1
    dense_buf = torch.einsum("sec,sm->ecm", sec, x.detach())
    assert torch.allclose(buf.view(E, C, H), dense_buf, atol=1e-6)
    cw = torch.zeros(S, E, C)
    for s in range(S):
        for k in range(K):
            if slot[s, k] >= 0:
                cw[s, slot[s, k] // C, slot[s, k] % C] = w[s, k].item()
    assert torch.allclose(y, torch.einsum("sec,ecm->sm", cw, dense_buf * 2.0), atol=1e-5)
    y.sum().backward()
    assert x.grad is not None and w.grad is not None


def _moe_model(seed=0):
    from oslo_b200.models.config import MoEGPTConfig
    from oslo_b200.models.gpt2 import MoEGPTLMHeadModel

    torch.manual_seed(seed)
    cfg = MoEGPTConfig(vocab_size=256, n_positions=32, n_embd=32, n_layer=2, n_head=4, resid_pdrop=0.0, embd_pdrop=0.0,
                       attn_pdrop=0.0, num_experts=4, moe_every=2, top_k=2)
    return MoEGPTLMHeadModel(cfg)


def _worker(rank, world, use_residual=False):
    import oslo_b200
    from oslo_b200 import ParallelContext
    from oslo_b200.parallel import ExpertParallel

    pc = ParallelContext.from_torch(expert_parallel_size=world, backend="gloo", seed=0)
    torch.manual_seed(7)
    ids_all = torch.randint(0, 256, (2 * world, 16))
    ids = ids_all.chunk(world)[rank]
    model = _moe_model()
    # large capacity: nothing is dropped, so routing is the same per token however the batch is split
    wrapped = ExpertParallel(model, pc, num_dec_experts={1: 4}, top_k=2, capacity_factor_train=8.0, use_rts=False,
                             aux_loss_coef=0.0, use_residual=use_residual)
    oslo_b200.ready(wrapped, pc)
    if use_residual:
        mixes = [n for n, _ in model.named_parameters() if "residual_mix" in n]
        dense = [n for n, _ in model.named_parameters() if ".residual." in n]
        assert len(mixes) == 2 and len(dense) >= 2, (mixes, dense)  # a 2-way mixer and dense copies of both linears
    wrapped.eval()  # no routing noise
    out = wrapped(input_ids=ids, labels=ids)
    out.loss.backward()
    loss = out.loss.detach().clone()
    torch.distributed.all_reduce(loss)
    loss /= world
    # single-group reference holding all experts on the whole batch
    from oslo_b200.parallel.expert_parallel.layers import Experts

    ref = _moe_model()
    ref_wrapped = ExpertParallel(ref, pc, num_dec_experts={1: 4}, top_k=2, capacity_factor_train=8.0, use_rts=False,
                                 aux_loss_coef=0.0, use_residual=use_residual)
    ref_wrapped.ep_size, ref_wrapped.ep_rank, ref_wrapped.sync_dense_grads = 1, 0, False
    ref_wrapped.parallelize()
    ref_wrapped.eval()
    losses = []
    for chunk in ids_all.chunk(world):
        o = ref_wrapped(input_ids=chunk, labels=chunk)
        (o.loss / world).backward()
        losses.append(o.loss.detach())
    ref_loss = torch.stack(losses).mean()
    assert torch.allclose(loss, ref_loss, rtol=1e-5, atol=1e-6), (loss.item(), ref_loss.item())
    ref_params = dict(ref.named_parameters())
    for name, p in model.named_parameters():
        r = ref_params[name]
        g = p.grad
        if getattr(p, "oslo_expert_param", False):
            e_local = p.shape[0]
            rg = r.grad[rank * e_local : (rank + 1) * e_local]
        else:
            rg = r.grad
        assert torch.allclose(g, rg, rtol=1e-4, atol=1e-6), (name, (g - rg).abs().max().item())
    pc.destroy()


def test_expert_parallel_matches_single_group():
    run_dist(_worker, 2)


def test_residual_moe_matches_single_group():
    """``use_residual=True``: a dense copy of the FFN runs beside the experts and a learned softmax mixes them."""
    run_dist(_worker, 2, True)


def test_gate_capacity_and_aux_loss():
    from oslo_b200.parallel.expert_parallel import TopKGate

    torch.manual_seed(1)
    gate = TopKGate(16, 4, k=1, capacity_factor=1.0, min_capacity=2, use_rts=False).eval()
    x = torch.randn(40, 16)
    l_aux, slot, weight, C = gate(x)
    assert C == 10
    assert (slot >= 0).sum() <= 4 * C
    per_expert = torch.bincount((slot[slot >= 0] // C).long(), minlength=4)
    assert per_expert.max() <= C
    assert l_aux.item() > 0
    kept = slot[slot >= 0]
    assert kept.unique().numel() == kept.numel()  # no two tokens share a buffer row


def _ep_tp_worker(rank, world, kind):
    """Expert x tensor parallelism (2 x 2 ranks): the experts are built from the whole feed-forward linears before the
    tensor-parallel wrapper shards the rest, which leaves routers and experts alone; the loss equals the expert-parallel-only
    model's."""
    import os
    import sys

    import oslo_b200
    from oslo_b200 import ParallelContext
    from oslo_b200.parallel import ExpertParallel, TensorParallel

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from test_tp_1d import _family

    pc = ParallelContext.from_torch(data_parallel_size=2, tensor_parallel_size=2, expert_parallel_size=2, backend="gloo", seed=0)
    model = _family(kind).train()
    ExpertParallel(model, pc, num_dec_experts=4, top_k=2, capacity_factor_train=4.0)
    TensorParallel(model, pc)
    oslo_b200.ready(model, pc)
    sharded = [n for n, p in model.named_parameters() if hasattr(p, "oslo_shard")]
    assert sharded and not any("gate" in n or "experts" in n for n in sharded), sharded
    ids = torch.randint(1, 100, (2, 12), generator=torch.Generator().manual_seed(1))
    out = model(input_ids=ids, labels=ids)
    out.loss.backward()
    ref = _family(kind).train()
    ExpertParallel(ref, pc, num_dec_experts=4, top_k=2, capacity_factor_train=4.0).parallelize()
    want = ref(input_ids=ids, labels=ids).loss
    assert abs(float(out.loss) - float(want)) < 1e-4, (kind, float(out.loss), float(want))
    pc.destroy()


@pytest.mark.parametrize("kind", ["gpt2", "neox"])
def test_expert_parallel_with_tensor_parallel(kind):
    run_dist(_ep_tp_worker, 4, kind)


def test_expert_parallel_refuses_pipeline_parallel():
    from oslo_b200.parallel import ExpertParallel

    class _PC:
        pipeline_parallel_size = 2

        def is_initialized(self, mode):
            return True

        def get_world_size(self, mode):
            return 2

        def get_local_rank(self, mode):
            return 0

    with pytest.raises(NotImplementedError, match="pipeline"):
        ExpertParallel(torch.nn.Linear(2, 2), _PC(), num_dec_experts=4)
