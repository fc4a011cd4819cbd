"""Time the row-sharded (ZeRO-3 style) linear with the parameter all-gather fused into its GEMM against the
all-gather + GEMM composition.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 \
        benchmarks/zero_linear_bench.py --tokens 8192 --in-features 2048 --out-features 8192

Per rank: ``tokens x in_features`` activations of its own batch, ``out_features / ranks`` rows of the weight.  Reported for
forward and for forward + backward: ``fused`` (``nn/zero_linear.py`` with the symmetric workspace of the DATA group enabled:
all-gather -> GEMM with the weight as the gathered operand, weight gradient through GEMM -> reduce-scatter) and
``composition`` (NCCL all-gather / reduce-scatter around the same products).  CUDA events on the launching stream, 3 warm-up
iterations, a barrier before each timed region, median of ``--iters``, MAX over ranks; operands and outputs together exceed
the 126 MB L2 at the default sizes.  Rank 0 prints a markdown table.
"""
from __future__ import annotations

import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--in-features", type=int, default=2048)
    ap.add_argument("--out-features", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

    from oslo_b200 import ParallelContext, ParallelMode
    from oslo_b200.distributed import symm
    from oslo_b200.nn.zero_linear import ZeroShardedLinear
    from oslo_b200.ops import _lib, fused_collectives as fc

    world = int(os.environ.get("WORLD_SIZE", "1"))
    pc = ParallelContext.from_torch(data_parallel_size=world, backend="nccl", seed=0)
    dev = pc.device
    torch.manual_seed(1)
    layer = ZeroShardedLinear(args.in_features, args.out_features, True, pc, dtype=torch.bfloat16, device=dev)
    x = (torch.randn(args.tokens, args.in_features, device=dev) * 0.5).to(torch.bfloat16)
    gy = (torch.randn(args.tokens, args.out_features, device=dev) * 0.1).to(torch.bfloat16)
    group = pc.get_group(ParallelMode.DATA)

    def fwd():
        with torch.no_grad():
            return layer(x)

    def fwd_bwd():
        xi = x.detach().requires_grad_(True)
        layer.weight.grad = layer.bias.grad = None
        layer(xi).backward(gy)

    def timed(fn):
        for _ in range(3):
            fn()
        times = []
        for _ in range(args.iters):
            torch.cuda.synchronize()
            dist.barrier(group=group)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            b.synchronize()
            times.append(a.elapsed_time(b))
        times.sort()
        t = torch.tensor([times[len(times) // 2]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        return float(t)

    rows = {"composition": (timed(fwd), timed(fwd_bwd))}
    from oslo_b200.nn import zero_linear as zl

    zl.FUSED_GATHER = True
    ok = symm.enable(pc, ParallelMode.DATA, max_tokens=args.out_features, max_features=max(args.in_features, args.tokens),
                     multimem=False)
    rt = fc.runtime(ParallelMode.DATA)
    if ok and rt is not None and rt.ws.ag_ok(layer.weight, x):
        before = rt.ws.epoch
        rows["fused"] = (timed(fwd), timed(fwd_bwd))
        assert rt.ws.epoch > before, "the fused kernels did not run"
    torch.cuda.synchronize()
    _lib.check_status()
    if pc.get_global_rank() == 0:
        flops_f = 2.0 * args.tokens * args.in_features * args.out_features
        gathered = (world - 1) / world * args.out_features * args.in_features * 2
        print(f"ranks {world}, tokens/rank {args.tokens}, in {args.in_features}, out {args.out_features}, bf16; "
              f"{gathered / 1e6:.1f} MB of weight rows arrive per rank and forward")
        print("| path | forward ms | TFLOP/s | forward + backward ms | TFLOP/s |")
        print("|---|---|---|---|---|")
        for name, (f, fb) in rows.items():
            print(f"| {name} | {f:.3f} | {flops_f / f / 1e9:.0f} | {fb:.3f} | {3 * flops_f / fb / 1e9:.0f} |")
        if "fused" in rows:
            print(f"fused / composition: forward {rows['composition'][0] / rows['fused'][0]:.2f}x, "
                  f"forward + backward {rows['composition'][1] / rows['fused'][1]:.2f}x")
    symm.disable()
    pc.destroy()


if __name__ == "__main__":
    main()
