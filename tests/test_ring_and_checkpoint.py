"""Ring self-attention over the SEQUENCE group and tensor-parallel partitioned activation checkpointing (CPU / gloo)."""
import torch

from dist_utils import run_dist


def _ring_worker(rank, world):
    from oslo_b200 import ParallelContext
    from oslo_b200.distributed import comm

    pc = ParallelContext.from_torch(sequence_parallel_size=world, backend="gloo", seed=0)
    torch.manual_seed(0)
    bh, s, d = 3, 8 * world, 16
    q = torch.randn(bh, s, d, requires_grad=True)
    k = torch.randn(bh, s, d, requires_grad=True)
    v = torch.randn(bh, s, d, requires_grad=True)
    scores = torch.matmul(q, k.transpose(1, 2)) / d ** 0.5
    out = torch.matmul(scores.softmax(-1), v)
    g = torch.randn(bh, s, d)
    out.backward(g)
    sl = s // world
    sub = lambda t: t.detach()[:, rank * sl : (rank + 1) * sl].clone().requires_grad_()
    ql, kl, vl = sub(q), sub(k), sub(v)
    sc = comm.ring_qk(ql, kl, pc) / d ** 0.5
    ol = comm.ring_av(sc.softmax(-1), vl, pc)
    assert torch.allclose(ol, out.detach()[:, rank * sl : (rank + 1) * sl], atol=1e-5)
    ol.backward(g[:, rank * sl : (rank + 1) * sl])
    for local, full in ((ql, q), (kl, k), (vl, v)):
        assert torch.allclose(local.grad, full.grad[:, rank * sl : (rank + 1) * sl], atol=1e-5)
    pc.destroy()


def test_ring_self_attention_matches_full_attention():
    run_dist(_ring_worker, 2)
    run_dist(_ring_worker, 4)


def _ckpt_worker(rank, world):
    import torch.nn as nn

    from oslo_b200 import ParallelContext
    from oslo_b200.utils.checkpoint import CheckpointFunction, CheckpointPartitioner

    pc = ParallelContext.from_torch(tensor_parallel_size=world, backend="gloo", seed=0)
    torch.manual_seed(0)
    layer = nn.Sequential(nn.Linear(12, 24), nn.Tanh(), nn.Linear(24, 12))
    x = torch.randn(5, 12, requires_grad=True)
    layer(x).sum().backward()
    want_x, want_w = x.grad.clone(), layer[0].weight.grad.clone()
    layer.zero_grad()
    x.grad = None
    part = CheckpointPartitioner(pc, partitioned=True, contiguous=True)
    kept, meta = part.partition([x])
    assert kept[0].numel() == 30  # 60 elements split over 2 tensor-parallel ranks
    y = CheckpointFunction.apply(layer, part, x)
    y.sum().backward()
    assert torch.allclose(x.grad, want_x, atol=1e-6) and torch.allclose(layer[0].weight.grad, want_w, atol=1e-6)
    pc.destroy()


def test_partitioned_activation_checkpointing():
    run_dist(_ckpt_worker, 2)
