"""Activation checkpointing (gradients equal the plain run, RNG replay), topology tables, P2P objects, logger."""
import pytest
import torch
import torch.nn as nn

from dist_utils import run_dist


def test_checkpoint_function_matches_plain_backward_with_dropout():
    from oslo_b200.utils.checkpoint import CheckpointFunction, CheckpointPartitioner

    torch.manual_seed(0)
    layer = nn.Sequential(nn.Linear(16, 32), nn.GELU(), nn.Dropout(0.3), nn.Linear(32, 16))
    x = torch.randn(4, 16, requires_grad=True)
    torch.manual_seed(5)
    y = layer(x)
    y.sum().backward()
    ref_gx = x.grad.clone()
    ref_gw = layer[0].weight.grad.clone()
    layer.zero_grad()
    x.grad = None
    torch.manual_seed(5)
    y2 = CheckpointFunction.apply(layer, CheckpointPartitioner(), x)
    torch.randn(3)  # disturb the RNG between forward and backward: the recomputation must replay the saved state
    y2.sum().backward()
    assert torch.allclose(y, y2) and torch.allclose(x.grad, ref_gx) and torch.allclose(layer[0].weight.grad, ref_gw)


@pytest.mark.parametrize("world", [1, 2, 4, 8, 16])
def test_topology_groups_partition_the_world(world):
    from oslo_b200.distributed import ParallelMode, Topology

    for tp, mode, depth in [(1, ParallelMode.TENSOR_1D, None), (2, ParallelMode.TENSOR_1D, None), (4, ParallelMode.TENSOR_2D, None),
                            (8, ParallelMode.TENSOR_2P5D, 2), (8, ParallelMode.TENSOR_3D, None)]:
        if world % tp:
            continue
        for pp in (1, 2):
            if (world // tp) % pp:
                continue
            dp = world // tp // pp
            topo = Topology(world, dp, pp, tp, 1, 1, mode, depth).validate()
            for m in topo.active_modes():
                groups = topo.groups(m)
                flat = sorted(r for g in groups for r in g)
                assert flat == list(range(world)), (m, groups)
                assert len({len(g) for g in groups}) == 1


def test_topology_reference_formulas():
    from oslo_b200.distributed import ParallelMode as M, Topology

    t = Topology(8, 2, 2, 2, 1, 1, M.TENSOR_1D).validate()
    assert t.groups(M.DATA) == [[0, 4], [1, 5], [2, 6], [3, 7]]
    assert t.groups(M.TENSOR) == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert t.groups(M.PIPELINE) == [[0, 2], [1, 3], [4, 6], [5, 7]]
    assert t.groups(M.MODEL) == [[0, 1, 2, 3], [4, 5, 6, 7]]
    t2 = Topology(4, 1, 1, 4, 1, 1, M.TENSOR_2D).validate()
    assert t2.groups(M.TENSOR_2D_ROW) == [[0, 1], [2, 3]] and t2.groups(M.TENSOR_2D_COL) == [[0, 2], [1, 3]]
    t3 = Topology(8, 1, 1, 8, 1, 1, M.TENSOR_3D).validate()
    assert t3.groups(M.TENSOR_3D_WEIGHT)[0] == [0, 1] and t3.groups(M.TENSOR_3D_INPUT)[0] == [0, 2]
    assert t3.groups(M.TENSOR_3D_OUTPUT)[0] == [0, 4]
    t25 = Topology(8, 1, 1, 8, 1, 1, M.TENSOR_2P5D, 2).validate()
    assert t25.groups(M.TENSOR_2P5D_DEP)[0] == [0, 4] and t25.groups(M.TENSOR_2P5D_XZ)[0] == [0, 2, 4, 6]
    ov = Topology(8, 8, 1, 1, 1, 8, M.TENSOR_1D, None, True).validate()
    assert ov.groups(M.EXPERT) == [list(range(8))]
    with pytest.raises(ValueError):
        Topology(8, 1, 1, 2, 2, 1, M.TENSOR_1D).validate()
    with pytest.raises(ValueError):
        Topology(6, 1, 1, 6, 1, 1, M.TENSOR_2D).validate()


def _p2p_worker(rank, world):
    from oslo_b200 import ParallelContext
    from oslo_b200.distributed import comm

    pc = ParallelContext.from_torch(data_parallel_size=world, backend="gloo")
    obj = {"a": [1, 2.5, "x", None, True], "t": torch.arange(6).view(2, 3).float(), "n": (torch.Size([2, 3]), {3, 4}),
           "g": torch.ones(2, requires_grad=True)}
    if rank == 0:
        comm.send(obj, 0, 1, parallel_context=pc)
    else:
        got = comm.recv(0, 1, parallel_context=pc)
        assert got["a"] == obj["a"] and torch.equal(got["t"], obj["t"]) and got["n"] == obj["n"]
        assert got["g"].requires_grad
    x = torch.full((2, 3), float(rank))
    g = comm.all_gather(x, dim=1, parallel_context=pc, parallel_mode=pc.topology and __import__("oslo_b200").ParallelMode.DATA)
    assert g.shape == (2, 3 * world) and g[0, 3].item() == 1.0
    pc.destroy()


def test_object_p2p_and_gather_dim():
    run_dist(_p2p_worker, 2)


def test_linear_cross_entropy_chunks_match_the_materialised_head():
    import torch
    import torch.nn.functional as F

    from oslo_b200.ops.linear_cross_entropy import linear_cross_entropy

    torch.manual_seed(0)
    T, H, V = 37, 16, 50
    hidden = torch.randn(3, T, H, requires_grad=True)
    weight = torch.randn(V, H, requires_grad=True)
    targets = torch.randint(0, V - 4, (3, T))
    targets[0, :5] = -100
    for chunk, valid in ((8, None), (1000, None), (16, V - 4)):
        hidden.grad = weight.grad = None
        loss = linear_cross_entropy(hidden, weight, targets, chunk_size=chunk, orig_vocab_size=valid)
        (loss * 2.0).backward()
        gh, gw = hidden.grad.clone(), weight.grad.clone()
        hidden.grad = weight.grad = None
        logits = hidden.reshape(-1, H) @ weight.t()
        if valid is not None:
            logits = logits[:, :valid]
        ref = F.cross_entropy(logits, targets.reshape(-1), ignore_index=-100)
        (ref * 2.0).backward()
        assert torch.allclose(loss, ref, atol=1e-5), (chunk, float(loss), float(ref))
        assert torch.allclose(gh, hidden.grad, atol=1e-5) and torch.allclose(gw, weight.grad, atol=1e-5), chunk


def test_documentation_names_exist():
    """Every ``oslo_b200...`` dotted name and every repository path quoted in the docs resolves (documentation that
    drifts from the code fails here)."""
    import importlib
    import os
    import re

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    docs = []
    for base, _, files in os.walk(os.path.join(root, "docs")):
        docs += [os.path.join(base, f) for f in files if f.endswith(".md")]
    assert len(docs) >= 10
    text = "\n".join(open(d, encoding="utf-8").read() for d in docs)
    for stmt in set(re.findall(r"^from (oslo_b200[\w.]*) import ([\w, ]+)$", text, flags=re.M)):
        mod = importlib.import_module(stmt[0])
        for name in stmt[1].split(","):
            name = name.strip().split(" as ")[0]
            if not hasattr(mod, name):
                importlib.import_module(f"{stmt[0]}.{name}")  # a submodule: ``from package import module``
    for path in set(re.findall(r"`((?:oslo_b200|examples|benchmarks|tests|profiles)/[\w/.{},*-]+\.(?:py|cu|cuh|cpp|md))`", text)):
        if any(c in path for c in "{*"):
            continue
        assert os.path.exists(os.path.join(root, path)), path
    for link in set(re.findall(r"\]\(([\w/._-]+\.md)\)", text)):
        assert any(os.path.exists(os.path.join(os.path.dirname(d), link)) for d in docs), link


def _launcher_worker(rank, world, kind, port):
    import os

    import torch
    import torch.distributed as dist

    from oslo_b200 import ParallelContext, ParallelMode

    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "LOCAL_WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT"):
        os.environ.pop(k, None)  # only the scheduler's own variables may be read
    if kind == "slurm":
        os.environ.update(SLURM_PROCID=str(rank), SLURM_NPROCS=str(world), SLURM_GPUS_ON_NODE=str(world))
        pc = ParallelContext.from_slurm("127.0.0.1", port, data_parallel_size=1, tensor_parallel_size=world, backend="gloo")
    else:
        os.environ.update(OMPI_COMM_WORLD_RANK=str(rank), OMPI_COMM_WORLD_LOCAL_RANK=str(rank), OMPI_COMM_WORLD_SIZE=str(world),
                          OMPI_COMM_WORLD_LOCAL_SIZE=str(world))
        pc = ParallelContext.from_openmpi("127.0.0.1", port, data_parallel_size=1, tensor_parallel_size=world, backend="gloo")
    assert pc.get_global_rank() == rank and pc.get_world_size(ParallelMode.GLOBAL) == world
    assert pc.get_world_size(ParallelMode.TENSOR) == world and pc.get_local_rank(ParallelMode.TENSOR) == rank
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t, group=pc.get_group(ParallelMode.TENSOR))
    assert float(t) == world * (world + 1) / 2
    pc.destroy()


def test_parallel_context_from_slurm_and_openmpi_variables():
    from dist_utils import free_port, run_dist

    for kind in ("slurm", "openmpi"):
        run_dist(_launcher_worker, 2, kind, free_port())
