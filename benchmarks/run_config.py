"""Device-timed training throughput for the multi-dimensional parallel configurations.

Launch with one rank per GPU, e.g.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29520 \
        benchmarks/run_config.py --config llama-2d-pp2 --steps 5 --warmup 3

Configurations (bf16, synthetic uniform token ids, random-init weights, AdamW):

    llama-2d-pp2   Llama-style 6.9B (32 layers, d 4096, 32 heads, SwiGLU 11008, vocab 32000), 2D tensor parallel 2x2 x
                   pipeline parallel 2, 1F1B with 8 micro-batches of 2 x 2048                         (8 GPUs)
    gpt-3d         GPT-style 2.7B (32 layers, d 2560, 32 heads, FFN 10240, vocab 50304), 3D tensor parallel 2x2x2,
                   global batch 16 x 2048                                                             (8 GPUs)
    gpt-2p5d       the same model, 2.5D tensor parallel (q = 2, depth = 2)                            (8 GPUs)
    moe-ep-zero2   MoE GPT (12 layers, d 1024, 16 heads, every other FFN = 16 experts of 4096, top-2, capacity factor
                   1.25, aux loss 0.01), expert parallel N + ZeRO-2 over the dense parameters, batch 32 x 1024 (N GPUs)

``--layers`` / ``--scale-down`` shrink a configuration for smoke runs on fewer GPUs; a shrunk run is labelled as such
in the output and is not a benchmark result.  Rank 0 prints one JSON line (tokens/s over the whole job, max over ranks).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def build(args, world):
    import oslo_b200
    from oslo_b200 import ParallelContext, ParallelMode
    from oslo_b200 import models
    from oslo_b200.optim import FusedAdam
    from oslo_b200.parallel import ExpertParallel, PipelineParallel, TensorParallel, ZeroRedundancyOptimizer

    name = args.config
    small = args.scale_down
    if name == "llama-2d-pp2":
        tp = args.tp or (4 if world >= 4 else 1)
        pp = world // tp
        pc = ParallelContext.from_torch(tensor_parallel_size=tp, pipeline_parallel_size=pp,
                                        tensor_parallel_mode=ParallelMode.TENSOR_2D, backend="nccl", seed=7)
        cfg = models.LlamaConfig(vocab_size=32000, hidden_size=1024 if small else 4096, intermediate_size=2816 if small else 11008,
                                 num_hidden_layers=args.layers or 32, num_attention_heads=8 if small else 32,
                                 max_position_embeddings=2048)
        batch, seq, micro = 16, 2048, 8
        cls = models.LlamaForCausalLM
    elif name in ("gpt-3d", "gpt-2p5d"):
        mode = ParallelMode.TENSOR_3D if name == "gpt-3d" else ParallelMode.TENSOR_2P5D
        depth = None if name == "gpt-3d" else (2 if world >= 8 else 1)
        pc = ParallelContext.from_torch(tensor_parallel_size=world, tensor_parallel_mode=mode, tensor_parallel_depth=depth,
                                        backend="nccl", seed=7)
        cfg = models.GPT2Config(vocab_size=50304, n_positions=2048, n_embd=1024 if small else 2560, n_layer=args.layers or 32,
                                n_head=16 if small else 32, n_inner=4096 if small else 10240, resid_pdrop=0.0, embd_pdrop=0.0,
                                attn_pdrop=0.0)
        batch, seq, micro = 16, 2048, 1
        cls = models.GPT2LMHeadModel
    elif name == "moe-ep-zero2":
        pc = ParallelContext.from_torch(data_parallel_size=world, expert_parallel_size=world, backend="nccl", seed=7)
        cfg = models.MoEGPTConfig(vocab_size=50304, n_positions=1024, n_embd=1024, n_layer=args.layers or 12, n_head=16,
                                  n_inner=4096, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0, num_experts=16, moe_every=2,
                                  top_k=2, capacity_factor=1.25, aux_loss_coef=0.01)
        batch, seq, micro = 32, 1024, 1
        cls = models.MoEGPTLMHeadModel
    else:
        raise SystemExit(f"unknown config {name}")
    dev = pc.device
    torch.manual_seed(7)
    with torch.device(dev):
        prev = torch.get_default_dtype()
        torch.set_default_dtype(torch.bfloat16)
        model = cls(cfg)
        torch.set_default_dtype(prev)
    wrapped = model
    if name == "moe-ep-zero2":
        layers = {i: cfg.num_experts for i in model.moe_layer_ids()}
        wrapped = ExpertParallel(model, pc, num_dec_experts=layers, top_k=cfg.top_k, capacity_factor_train=cfg.capacity_factor,
                                 aux_loss_coef=cfg.aux_loss_coef, sync_dense_grads=False)
    else:
        if pc.tensor_parallel_size > 1:
            wrapped = TensorParallel(model, pc)
        if pc.pipeline_parallel_size > 1:
            wrapped = PipelineParallel(model, pc, num_micro_batches=micro)
    oslo_b200.ready(wrapped, pc)
    fused = []
    if not args.no_fused:
        from oslo_b200.distributed import symm

        M = ParallelMode
        tokens = batch * seq // max(micro, 1)
        widest = max(getattr(cfg, "intermediate_size", 0) * 2, getattr(cfg, "n_inner", 0) or 0, 3 * getattr(cfg, "hidden_size", getattr(cfg, "n_embd", 0)))
        if name == "llama-2d-pp2" and pc.tensor_parallel_size > 1:
            rows = tokens // pc.summa_dim  # every rank keeps its share of the micro-batch
            fused += [M.TENSOR_2D_ROW] if symm.enable(pc, M.TENSOR_2D_ROW, rows, widest) else []
        elif name == "gpt-2p5d":
            rows = tokens // (pc.summa_dim * (pc.tensor_parallel_depth or 1))
            fused += [M.TENSOR_2P5D_ROW] if symm.enable(pc, M.TENSOR_2P5D_ROW, rows, widest) else []
        elif name == "gpt-3d":
            rows = tokens // pc.cubic_dim  # rows of the product after the INPUT gather
            for mode in (M.TENSOR_3D_INPUT, M.TENSOR_3D_OUTPUT):
                fused += [mode] if symm.enable(pc, mode, rows, widest // pc.cubic_dim if mode == M.TENSOR_3D_OUTPUT else widest) else []
        elif name == "moe-ep-zero2":
            symm._fused_small_ops = True  # expert dispatch / combine through peer memory, fused ZeRO step
            fused += ["moe-peer-dispatch", "zero-step"]
    args.fused_paths = [str(f) for f in fused]
    params = [p for p in model.parameters() if p.requires_grad and p.numel() > 0]
    if name == "moe-ep-zero2":
        dense = [p for p in params if not getattr(p, "oslo_expert_param", False)]
        experts = [p for p in params if getattr(p, "oslo_expert_param", False)]
        zero = ZeroRedundancyOptimizer(torch.optim.AdamW(dense, lr=1e-4, weight_decay=0.01), parallel_context=pc,
                                       partition_grad=True, fused=not args.no_fused, overlap_communication=not args.no_fused)
        expert_opt = FusedAdam(experts, lr=1e-4, weight_decay=0.01, master_weights=True)
        opts = (zero, expert_opt)
    else:
        opts = (FusedAdam(params, lr=1e-4, weight_decay=0.01, master_weights=True),)
    return pc, model, wrapped, opts, cfg, batch, seq


def flops_per_token(name, cfg, seq) -> float:
    """Training FLOPs per token: 6 x (matrix parameters a token passes through) + causal attention."""
    h = getattr(cfg, "hidden_size", None) or cfg.n_embd
    L = getattr(cfg, "num_hidden_layers", None) or cfg.n_layer
    v = cfg.vocab_size
    if name == "llama-2d-pp2":
        per_layer = [4 * h * h + 3 * h * cfg.intermediate_size] * L
    elif name == "moe-ep-zero2":
        f = cfg.n_inner
        moe = set(range(L)[1::2]) if cfg.moe_every == 2 else set()
        per_layer = [4 * h * h + (cfg.top_k * 2 * h * f if i in moe else 2 * h * f) for i in range(L)]
    else:
        per_layer = [4 * h * h + 2 * h * cfg.n_inner] * L
    return 6.0 * (sum(per_layer) + h * v) + L * 6.0 * seq * h


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, choices=["llama-2d-pp2", "gpt-3d", "gpt-2p5d", "moe-ep-zero2"])
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--scale-down", action="store_true")
    ap.add_argument("--no-fused", action="store_true",
                    help="run the NCCL collective + GEMM compositions instead of the fused peer-memory kernels")
    ap.add_argument("--tp", type=int, default=0, help="override the tensor-parallel size of llama-2d-pp2 (smoke runs)")
    args = ap.parse_args()
    world = int(os.environ["WORLD_SIZE"])
    pc, model, wrapped, opts, cfg, batch, seq = build(args, world)
    from oslo_b200 import ParallelMode
    from oslo_b200.ops import _lib

    dev = pc.device
    rank = pc.get_global_rank()
    gen = torch.Generator().manual_seed(3)
    vocab = cfg.vocab_size
    dp = pc.get_world_size(ParallelMode.DATA)
    dp_rank = pc.get_local_rank(ParallelMode.DATA)
    batches = [torch.randint(0, vocab, (batch, seq), generator=gen) for _ in range(4)]
    local = [b.chunk(dp)[dp_rank].to(dev) for b in batches]
    is_pp = pc.pipeline_parallel_size > 1
    zero = opts[0] if hasattr(opts[0], "backward") else None

    def step(ids):
        for o in opts:
            o.zero_grad()
        if is_pp:
            total = None
            for _, out in wrapped(input_ids=ids, labels=ids):
                if torch.is_tensor(out.loss):
                    out.loss.backward()
                    total = out.loss.detach() if total is None else total + out.loss.detach()
            loss = total
        else:
            loss = wrapped(input_ids=ids, labels=ids).loss
            if zero is not None:
                zero.backward(loss)
            else:
                loss.backward()
        for o in opts:
            o.step()
        return loss

    for i in range(max(3, args.warmup)):
        step(local[i % 4])
    torch.cuda.synchronize()
    _lib.check_status()
    dist.barrier()
    from bench import ClockSampler  # NVML reader of the flagship benchmark (read-only)

    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    last = None
    for i in range(args.steps):
        last = step(local[i % 4])
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    _lib.check_status()
    clocks = sampler.stop()
    ms = t.item() / args.steps
    lossv = torch.tensor([float(last) if last is not None else 0.0], device=dev)
    dist.all_reduce(lossv, op=dist.ReduceOp.MAX)
    if rank == 0:
        nparams = sum(p.numel() for p in model.parameters())
        print(json.dumps({
            "metric": "train tokens/sec (device-timed, max over ranks)", "config": args.config, "value": batch * seq / (ms / 1e3),
            "unit": "tokens/s", "n_gpus": world, "ms_per_step": ms, "steps": args.steps, "global_batch": batch, "seq_len": seq,
            "dtype": "bf16", "data": "synthetic", "rank_local_params": nparams, "loss": lossv.item(),
            "shrunk": bool(args.layers or args.scale_down), "fused_paths": args.fused_paths, "clocks": clocks,
            "per_gpu_model_tflops": batch * seq / (ms / 1e3) * flops_per_token(args.config, cfg, seq) / 1e12 / world,
            "parallelism": dict(tp=pc.tensor_parallel_size, pp=pc.pipeline_parallel_size, dp=pc.data_parallel_size,
                                ep=pc.expert_parallel_size if isinstance(pc.expert_parallel_size, int) else 0,
                                mode=str(pc.tensor_parallel_mode)),
        }))
    dist.barrier()
    pc.destroy()


if __name__ == "__main__":
    main()
