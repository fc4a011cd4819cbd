"""Fused all-gather->GEMM and GEMM->reduce-scatter kernels vs the NCCL + matmul composition (needs >= 2 GPUs)."""
import os

import pytest
import torch

from dist_utils import run_dist

pytestmark = pytest.mark.gpu


def _n_gpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _worker(rank, world, multimem=False, ce=False):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["OSLO_B200_MULTIMEM_MIN_RANKS"] = "2"  # exercise the multicast kernels on two ranks as well
    import torch.distributed as dist

    from oslo_b200 import ParallelContext, ParallelMode
    from oslo_b200.distributed import comm, symm
    from oslo_b200.ops import _lib, fused_collectives as fc

    pc = ParallelContext.from_torch(tensor_parallel_size=world, tensor_parallel_mode=ParallelMode.TENSOR_1D,
                                    backend="nccl", seed=0)
    dev = pc.device
    # multimem: the workspace is bound to an NVSwitch multicast object when the box allows it (the all-gather then uses
    # multimem.st, the row reduce-scatter multimem.ld_reduce); otherwise, and with multimem off, plain peer stores
    assert symm.enable(pc, ParallelMode.TENSOR_1D, max_tokens=4096, max_features=1024, multimem=multimem, ce_transport=ce)
    assert fc.runtime().ws.ce_transport == ce
    if multimem and rank == 0:
        print(f"multicast workspace: {'bound' if fc.runtime().ws.mc_base else 'not available (' + str(symm._multicast_alloc.last_error) + ')'}",
              flush=True)
    # a second workspace over the same ranks stands for the second group of the 3-D linear (gather and scatter groups
    # differ there; the kernel only sees two sets of peer pointers, flags and epochs)
    ws2 = symm.SymmetricWorkspace(pc, ParallelMode.TENSOR_1D, 4096, 1024)
    M1 = ParallelMode.TENSOR_1D
    torch.manual_seed(100 + rank)

    def rel(a, b):
        return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)

    for it, (T, K, N, b_t) in enumerate([(1024, 512, 384, False), (2048, 1024, 768, True), (1024, 256, 1024, False),
                                          (4096, 1024, 256, True), (1024, 512, 384, False)]):
        tl = T // world
        # ---- all-gather -> GEMM
        x = (torch.randn(tl, K, device=dev) * 0.5).to(torch.bfloat16)
        w = (torch.randn(K, N, device=dev) * 0.1).to(torch.bfloat16) if b_t else (torch.randn(N, K, device=dev) * 0.1).to(torch.bfloat16)
        W = w.t() if b_t else w
        assert fc.available(x, W, "ag")
        y, x_full = fc.ag_gemm(x, W, pc)
        x_ref = comm.all_gather(x, dim=0, parallel_context=pc, parallel_mode=M1)
        y_ref = x_ref.float() @ W.float().t()
        torch.cuda.synchronize()
        _lib.check_status()
        assert torch.equal(x_full, x_ref), f"gathered activations differ (case {it})"
        assert rel(y, y_ref) < 1e-2, (it, rel(y, y_ref))
        # ---- GEMM -> reduce-scatter
        xa = (torch.randn(T, K, device=dev) * 0.5).to(torch.bfloat16)
        wn = (torch.randn(K, N, device=dev) * 0.1).to(torch.bfloat16) if b_t else (torch.randn(N, K, device=dev) * 0.1).to(torch.bfloat16)
        WN = wn.t() if b_t else wn
        assert fc.available(xa, WN, "rs")
        out = fc.gemm_rs(xa, WN, pc)
        part = (xa.float() @ WN.float().t())
        ref = comm.reduce_scatter(part, dim=0, parallel_context=pc, parallel_mode=M1)
        torch.cuda.synchronize()
        _lib.check_status()
        assert rel(out, ref) < 2e-2, (it, rel(out, ref))
        # ---- the same with a local [T, N] addend riding along (two row products, one reduce-scatter)
        add = (torch.randn(T, N, device=dev) * 0.5).to(torch.bfloat16)
        out2 = fc.gemm_rs(xa, WN, pc, addend=add)
        ref2 = comm.reduce_scatter(part + add.float(), dim=0, parallel_context=pc, parallel_mode=M1)
        torch.cuda.synchronize()
        _lib.check_status()
        assert rel(out2, ref2) < 2e-2, (it, rel(out2, ref2))
        # ---- the same with the second product given as operands (x', w') instead of a ready addend
        k2 = 256
        xb = (torch.randn(T, k2, device=dev) * 0.5).to(torch.bfloat16)
        wb = (torch.randn(N, k2, device=dev) * 0.1).to(torch.bfloat16)
        out2b = fc.gemm_rs(xa, WN, pc, pair=(xb, wb))
        ref2b = comm.reduce_scatter(part + xb.float() @ wb.float().t(), dim=0, parallel_context=pc, parallel_mode=M1)
        torch.cuda.synchronize()
        _lib.check_status()
        assert rel(out2b, ref2b) < 2e-2, (it, rel(out2b, ref2b))
        # ---- reduce-scatter along the FEATURE dim (2-D / 2.5-D layouts): every rank keeps its rows
        ws = fc.runtime().ws
        if ws.rs_ok(xa, WN, along_n=True):
            out3 = ws.gemm_rs(xa, WN, along_n=True)
            ref3 = comm.reduce_scatter(part, dim=-1, parallel_context=pc, parallel_mode=M1)
            torch.cuda.synchronize()
            _lib.check_status()
            assert out3.shape == ref3.shape, (out3.shape, ref3.shape)
            assert rel(out3, ref3) < 2e-2, (it, rel(out3, ref3))
        # ---- all-gather (one workspace) -> GEMM -> reduce-scatter of the rows (a second workspace) in one launch
        out4, xf4 = ws.ag_gemm_rs(ws2, x, W)
        ref4 = comm.reduce_scatter(y_ref, dim=0, parallel_context=pc, parallel_mode=M1)
        torch.cuda.synchronize()
        _lib.check_status()
        assert torch.equal(xf4, x_ref), f"gathered activations differ in the gather+scatter launch (case {it})"
        assert rel(out4, ref4) < 2e-2, (it, rel(out4, ref4))
    dist.barrier()
    pc.destroy()


def _world_sizes():
    """Every power of two up to the number of visible GPUs (2, 4, 8): the 8-rank case runs wherever 8 GPUs are."""
    return [w for w in (2, 4, 8) if w <= _n_gpus()] or [2]


@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("transport", ["peer", "multicast", "copy-engine"])
@pytest.mark.parametrize("world", _world_sizes())
def test_fused_collectives_match_nccl(world, transport):
    """peer: copy CTAs / epilogue stores inside the kernel; multicast: multimem.st / multimem.ld_reduce; copy-engine: the
    shards travel by cudaMemcpyAsync between peer mappings on side streams while every SM multiplies."""
    run_dist(_worker, world, transport == "multicast", transport == "copy-engine", timeout=600)


def _model_worker(rank, world):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import oslo_b200
    from oslo_b200 import ParallelContext, ParallelMode
    from oslo_b200.distributed import symm
    from oslo_b200.models.config import GPTNeoXConfig
    from oslo_b200.models.gpt_neox import GPTNeoXForCausalLM
    from oslo_b200.ops import _lib
    from oslo_b200.parallel import TensorParallel

    pc = ParallelContext.from_torch(tensor_parallel_size=world, tensor_parallel_mode=ParallelMode.TENSOR_1D,
                                    backend="nccl", seed=0)
    dev = pc.device
    cfg = GPTNeoXConfig(vocab_size=2048, hidden_size=512, num_hidden_layers=2, num_attention_heads=8,
                        intermediate_size=2048, max_position_embeddings=256)
    losses = {}
    grads = {}
    for fused in (False, True):
        torch.manual_seed(3)
        model = GPTNeoXForCausalLM(cfg).to(dev, torch.bfloat16)
        wrapped = TensorParallel(model, pc, sequence_parallel=True)
        oslo_b200.ready(wrapped, pc)
        if fused:
            assert symm.enable(pc, ParallelMode.TENSOR_1D, max_tokens=world * 2 * 256, max_features=512)
        else:
            symm.disable()
        torch.manual_seed(4)
        ids = torch.randint(0, 2048, (world * 2, 256), device=dev)
        loss = wrapped(input_ids=ids, labels=ids).loss
        loss.backward()
        torch.cuda.synchronize()
        _lib.check_status()
        losses[fused] = loss.item()
        grads[fused] = {k: p.grad.float().clone() for k, p in model.named_parameters()}
    assert abs(losses[True] - losses[False]) < 2e-2, losses
    for k in grads[True]:
        a, b = grads[True][k], grads[False][k]
        assert (a - b).abs().max().item() <= 5e-2 * (b.abs().max().item() + 1e-3), k
    symm.disable()
    pc.destroy()


@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
def test_fused_model_step_matches_composition():
    run_dist(_model_worker, 2, timeout=600)


def _zero_worker(rank, world, clip):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.nn as nn

    from oslo_b200 import ParallelContext, ParallelMode
    from oslo_b200.distributed import symm
    from oslo_b200.ops import _lib
    from oslo_b200.parallel import ZeroRedundancyOptimizer

    pc = ParallelContext.from_torch(data_parallel_size=world, backend="nccl", seed=0)
    dev = pc.device

    def make():
        torch.manual_seed(0)
        return nn.Sequential(nn.Linear(256, 512), nn.GELU(), nn.Linear(512, 512), nn.LayerNorm(512), nn.Linear(512, 64)).to(dev, torch.bfloat16)

    results = {}
    for fused in (False, True, "overlap"):
        model = make()
        opt = ZeroRedundancyOptimizer(torch.optim.AdamW(model.parameters(), lr=1e-2, weight_decay=0.1), parallel_context=pc,
                                      partition_grad=True, fused=bool(fused), clip_grad_norm=clip,
                                      overlap_communication=fused == "overlap", reduce_bucket_size=64 * 1024)
        assert opt.fused == bool(fused)
        if fused:
            assert sum(len(g.buckets) for g in opt._all_groups()) > 2  # several per-bucket kernels
        for s in range(3):
            g = torch.Generator().manual_seed(10 + s)
            x = torch.randn(8 * world, 256, generator=g).to(dev, torch.bfloat16).chunk(world)[rank]
            y = torch.randn(8 * world, 64, generator=g).to(dev, torch.bfloat16).chunk(world)[rank]
            opt.zero_grad()
            loss = ((model(x) - y).float() ** 2).mean()
            opt.backward(loss)
            opt.step()
        torch.cuda.synchronize()
        _lib.check_status()
        results[fused] = [p.detach().float().clone() for p in model.parameters()]
    bad = []
    for key in (True, "overlap"):
        for i, (a, b) in enumerate(zip(results[key], results[False])):
            # AdamW moves a weight by about lr whatever the size of its gradient, so the handful of elements whose two
            # per-rank gradients nearly cancel (bf16 sum in the collective path, fp32 sum in the kernel) may differ by a
            # step; everything else must agree closely
            tol = 2e-2 * (b.abs().max().item() + 1e-3)
            err = (a - b).abs()
            frac = (err > tol).float().mean().item()
            if frac > 1e-3 or err.max().item() > 3 * 1e-2 * 3:
                bad.append((key, i, tuple(a.shape), err.max().item(), tol, frac))
    assert not bad, bad
    pc.destroy()


@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("clip", [1.0, 0.0])
def test_fused_zero_step_matches_collective_path(clip):
    run_dist(_zero_worker, 2, clip, timeout=600)


def _moe_worker(rank, world):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import oslo_b200
    from oslo_b200 import ParallelContext, ParallelMode
    from oslo_b200.distributed import symm
    from oslo_b200.models import MoEGPTConfig, MoEGPTLMHeadModel
    from oslo_b200.ops import _lib
    from oslo_b200.parallel import ExpertParallel

    pc = ParallelContext.from_torch(expert_parallel_size=world, backend="nccl", seed=0)
    dev = pc.device
    cfg = MoEGPTConfig(vocab_size=512, n_positions=64, n_embd=128, n_layer=2, n_head=4, resid_pdrop=0.0, embd_pdrop=0.0,
                       attn_pdrop=0.0, num_experts=4, moe_every=2, top_k=2)
    res = {}
    for fused in (False, True):
        torch.manual_seed(0)
        model = MoEGPTLMHeadModel(cfg).to(dev, torch.bfloat16)
        wrapped = ExpertParallel(model, pc, num_dec_experts={1: 4}, top_k=2, capacity_factor_train=2.0, use_rts=False)
        oslo_b200.ready(wrapped, pc)
        wrapped.eval()
        symm._fused_small_ops = fused
        torch.manual_seed(5 + rank)
        ids = torch.randint(0, 512, (2, 64), device=dev)
        loss = wrapped(input_ids=ids, labels=ids).loss
        loss.backward()
        torch.cuda.synchronize()
        _lib.check_status()
        res[fused] = (loss.item(), {k: p.grad.float().clone() for k, p in model.named_parameters() if p.grad is not None})
    symm._fused_small_ops = False
    assert abs(res[True][0] - res[False][0]) < 2e-2, (res[True][0], res[False][0])
    for k, g in res[False][1].items():
        a = res[True][1][k]
        assert (a - g).abs().max().item() <= 6e-2 * (g.abs().max().item() + 1e-3), k
    pc.destroy()


@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
def test_moe_peer_dispatch_combine_matches_all_to_all():
    run_dist(_moe_worker, 2, timeout=600)


def _nd_worker(rank, world, mode_name):
    """2-D / 2.5-D / 3-D tensor parallel model step: fused kernels (feature reduce-scatter, gather + GEMM + scatter)
    against the NCCL collective + GEMM compositions of the same layers."""
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import oslo_b200
    from oslo_b200 import ParallelContext, ParallelMode
    from oslo_b200 import models
    from oslo_b200.distributed import symm
    from oslo_b200.ops import _lib
    from oslo_b200.parallel import TensorParallel

    M = ParallelMode
    mode = getattr(M, mode_name)
    depth = 2 if (mode == M.TENSOR_2P5D and world == 8) else (1 if mode == M.TENSOR_2P5D else None)
    pc = ParallelContext.from_torch(tensor_parallel_size=world, tensor_parallel_mode=mode, tensor_parallel_depth=depth,
                                    backend="nccl", seed=0)
    dev = pc.device
    cfg = models.GPT2Config(vocab_size=2048, n_positions=256, n_embd=512, n_layer=2, n_head=8, n_inner=2048, resid_pdrop=0.0,
                            embd_pdrop=0.0, attn_pdrop=0.0)
    res = {}
    for fused in (False, True):
        torch.manual_seed(3)
        model = models.GPT2LMHeadModel(cfg).to(dev, torch.bfloat16)
        wrapped = TensorParallel(model, pc)
        oslo_b200.ready(wrapped, pc)
        symm.disable()
        if fused:
            rows, widest = 8 * 256, 3 * 512
            if mode == M.TENSOR_3D:
                assert symm.enable(pc, M.TENSOR_3D_INPUT, rows, widest) and symm.enable(pc, M.TENSOR_3D_OUTPUT, rows, widest)
            else:
                assert symm.enable(pc, M.TENSOR_2D_ROW if mode == M.TENSOR_2D else M.TENSOR_2P5D_ROW, rows, widest)
        torch.manual_seed(4)
        ids = torch.randint(0, 2048, (8, 256), device=dev)
        loss = wrapped(input_ids=ids, labels=ids).loss
        loss.backward()
        torch.cuda.synchronize()
        _lib.check_status()
        res[fused] = (loss.item(), {k: p.grad.float().clone() for k, p in model.named_parameters() if p.grad is not None})
    symm.disable()
    assert abs(res[True][0] - res[False][0]) < 2e-2, (res[True][0], res[False][0])
    for k, g in res[False][1].items():
        a = res[True][1][k]
        assert (a - g).abs().max().item() <= 5e-2 * (g.abs().max().item() + 1e-3), k
    pc.destroy()


@pytest.mark.skipif(_n_gpus() < 4, reason="needs at least 4 GPUs")
@pytest.mark.parametrize("mode", ["TENSOR_2D", "TENSOR_2P5D"])
def test_fused_2d_model_step_matches_composition(mode):
    run_dist(_nd_worker, 4, mode, timeout=600)


@pytest.mark.skipif(_n_gpus() < 8, reason="needs 8 GPUs")
def test_fused_3d_model_step_matches_composition():
    run_dist(_nd_worker, 8, "TENSOR_3D", timeout=600)


def _zero_linear_worker(rank, world):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from oslo_b200 import ParallelContext, ParallelMode
    from oslo_b200.distributed import symm
    from oslo_b200.nn.zero_linear import ZeroShardedLinear
    from oslo_b200.ops import _lib, fused_collectives as fc

    pc = ParallelContext.from_torch(data_parallel_size=world, backend="nccl", seed=0)
    dev = pc.device
    torch.manual_seed(7)  # same full layer on every rank
    full = torch.nn.Linear(256, 512).to(dev, torch.bfloat16)
    layer = ZeroShardedLinear.from_linear(full, pc)
    torch.manual_seed(50 + rank)  # own batch per rank
    x = (torch.randn(4, 256, 256, device=dev) * 0.5).to(torch.bfloat16)
    gy = (torch.randn(4, 256, 512, device=dev) * 0.1).to(torch.bfloat16)

    def run():
        xi = x.clone().requires_grad_(True)
        layer.weight.grad = layer.bias.grad = None
        y = layer(xi)
        y.backward(gy)
        torch.cuda.synchronize()
        _lib.check_status()
        return y.detach().float().clone(), xi.grad.float().clone(), layer.weight.grad.float().clone(), layer.bias.grad.float().clone()

    ref = run()  # collective + matmul composition: no workspace yet
    from oslo_b200.nn import zero_linear as zl

    zl.FUSED_GATHER = True  # the fused route is opt-in (measured slower than the composition at this size)
    assert symm.enable(pc, ParallelMode.DATA, max_tokens=1024, max_features=1024, multimem=False)
    rt = fc.runtime(ParallelMode.DATA)
    assert rt is not None and rt.ws.ag_ok(layer.weight, x.reshape(-1, 256))
    before = rt.ws.epoch
    got = run()
    assert rt.ws.epoch >= before + 2, "the fused all-gather GEMM and GEMM reduce-scatter did not run"
    for name, a, b in zip(("y", "dx", "dw", "db"), got, ref):
        err = (a - b).abs().max().item() / (b.abs().max().item() + 1e-6)
        assert err < 2e-2, (name, err)
    symm.disable()
    pc.destroy()


@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
def test_zero_sharded_linear_fused_gather_gemm_matches_composition():
    run_dist(_zero_linear_worker, 2, timeout=600)
