"""Time the fused compute + collective kernels of the sequence-parallel linears against their NCCL compositions.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29531 \
        benchmarks/fused_collective_bench.py --tokens 16384 --hidden 2048 --ffn 8192

For every linear of a GPT-NeoX-style block at the given tensor-parallel size (= the number of ranks) it reports

* ``fused``      one launch of ``oslo_ag_gemm`` / ``oslo_gemm_rs`` (peer loads / TMA stores to peer memory inside the GEMM);
* ``nccl+gemm``  ``all_gather_into_tensor`` + the same tcgen05 GEMM, or that GEMM + ``reduce_scatter_tensor``;
* ``gemm``       the GEMM alone, on already gathered data (the compute floor);
* the roofline: the slower of FLOPs / measured bf16 peak and bytes-that-must-cross-NVLink / 770 GB/s per direction,
  and ``fused`` as a fraction of it.

Timing: CUDA events on the launching stream, 3 warm-up launches, a barrier before each timed region, an L2 flush
between regions, median of ``--iters``, MAX over ranks; ``--inner`` calls per region (1: an isolated call, including the
skew between ranks after the barrier; more: the steady state inside a training step).  Rank 0 prints a markdown table.
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

LINK_GBS = 770.0  # measured peer copy, per direction per GPU


def peak_tflops():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f)["bf16_tflops"], "measured"
    except Exception:
        return 1590.0, "fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--copy-ctas", type=int, default=None)
    ap.add_argument("--inner", type=int, default=1,
                    help="calls issued back to back per timed region (times are per call): 1 shows an isolated call including "
                         "the skew between ranks after the barrier, larger values the steady state inside a step")
    ap.add_argument("--ce", action="store_true", help="copy-engine transport (cudaMemcpyAsync on side streams, every SM multiplies)")
    ap.add_argument("--no-multimem", action="store_true", help="plain peer stores even where NVSwitch multicast is available")
    args = ap.parse_args()

    from oslo_b200 import ParallelContext, ParallelMode
    from oslo_b200.distributed import symm
    from oslo_b200.ops import _lib, fused_collectives as fc
    from oslo_b200.ops.gemm import matmul_nt

    world = int(os.environ["WORLD_SIZE"])
    pc = ParallelContext.from_torch(tensor_parallel_size=world, tensor_parallel_mode=ParallelMode.TENSOR_1D,
                                    backend="nccl", seed=0)
    dev, rank = pc.device, pc.get_global_rank()
    group = pc.get_group(ParallelMode.TENSOR_1D)
    T, H, F = args.tokens, args.hidden, args.ffn
    kw = {} if args.copy_ctas is None else {"copy_ctas": args.copy_ctas}
    kw["multimem"] = not args.no_multimem and not args.ce
    kw["ce_transport"] = args.ce
    assert symm.enable(pc, ParallelMode.TENSOR_1D, max_tokens=T, max_features=max(H, F // world, 3 * H // world), **kw)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    tl = T // world
    peak, src = peak_tflops()

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(args.iters):
            flush.zero_()
            dist.barrier(group=group)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.inner):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / args.inner)
        ts.sort()
        t = torch.tensor([ts[len(ts) // 2]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        return t.item()

    def rnd(*shape):
        return (torch.randn(*shape, device=dev) * 0.1).to(torch.bfloat16)

    rows = []
    # (name, kind, K, N): column linears gather tokens first, row linears reduce-scatter them afterwards
    cases = [("qkv (AG->GEMM)", "ag", H, 3 * H // world), ("h_to_4h (AG->GEMM)", "ag", H, F // world),
             ("qkv + h_to_4h (one AG, two GEMMs)", "ag2", H, (3 * H + F) // world),
             ("dense (GEMM->RS)", "rs", H // world, H), ("4h_to_h (GEMM->RS)", "rs", F // world, H),
             ("dense + 4h_to_h (one RS)", "rs2", (H + F) // world, H)]
    for name, kind, K, N in cases:
        flops = 2.0 * T * K * N
        link_bytes = (world - 1) / world * T * (K if kind.startswith("ag") else N) * 2
        roof_ms = max(flops / (peak * 1e9), link_bytes / (LINK_GBS * 1e6))
        if kind == "ag":
            x, w = rnd(tl, K), rnd(N, K)
            x_full = torch.empty(T, K, dtype=torch.bfloat16, device=dev)
            fused = timed(lambda: fc.ag_gemm(x, w, pc, keep=False))

            def comp():
                dist.all_gather_into_tensor(x_full, x, group=group)
                return matmul_nt(x_full, w)

            nccl = timed(comp)
            alone = timed(lambda: matmul_nt(x_full, w))
        elif kind == "ag2":
            n1 = 3 * H // world
            x, w1, w2 = rnd(tl, K), rnd(n1, K), rnd(N - n1, K)
            x_full = torch.empty(T, K, dtype=torch.bfloat16, device=dev)

            def fused_fn():
                y1, xf = fc.ag_gemm(x, w1, pc, keep=False)
                return y1, matmul_nt(xf, w2)

            def comp():
                dist.all_gather_into_tensor(x_full, x, group=group)
                return matmul_nt(x_full, w1), matmul_nt(x_full, w2)

            fused, nccl = timed(fused_fn), timed(comp)
            alone = timed(lambda: (matmul_nt(x_full, w1), matmul_nt(x_full, w2)))
        elif kind == "rs":
            x, w = rnd(T, K), rnd(N, K)
            out = torch.empty(tl, N, dtype=torch.bfloat16, device=dev)
            fused = timed(lambda: fc.gemm_rs(x, w, pc))

            def comp():
                dist.reduce_scatter_tensor(out, matmul_nt(x, w), group=group)

            nccl = timed(comp)
            alone = timed(lambda: matmul_nt(x, w))
        else:
            k1 = H // world
            x1, w1, x2, w2 = rnd(T, k1), rnd(N, k1), rnd(T, K - k1), rnd(N, K - k1)
            out = torch.empty(tl, N, dtype=torch.bfloat16, device=dev)
            fused = timed(lambda: fc.gemm_rs(x2, w2, pc, pair=(x1, w1)))

            def comp():
                dist.reduce_scatter_tensor(out, matmul_nt(x1, w1) + matmul_nt(x2, w2), group=group)

            nccl = timed(comp)
            alone = timed(lambda: (matmul_nt(x1, w1), matmul_nt(x2, w2)))
        torch.cuda.synchronize()
        _lib.check_status()
        rows.append((name, K, N, fused, nccl, alone, roof_ms, roof_ms / fused))
    if rank == 0:
        ws = fc.runtime().ws
        print(f"transport: {'copy engine' if ws.ce_transport else 'NVSwitch multicast (multimem.st / multimem.ld_reduce)' if ws.mc_base else 'peer stores'}"
              + ("" if ws.mc_base or args.no_multimem else f" (multicast not available: {symm._multicast_alloc.last_error})")
              + f", {ws.copy_ctas} copy / reduce CTAs")
        print(f"tp = {world}, tokens = {T}, hidden = {H}, ffn = {F}; bf16; roofline = max(FLOPs / {peak:.0f} TFLOP/s ({src}), "
              f"NVLink bytes / {LINK_GBS:.0f} GB/s)")
        print("| op | K | N | fused ms | NCCL + GEMM ms | GEMM alone ms | roofline ms | fused / roofline |")
        print("|---|---|---|---|---|---|---|---|")
        for name, K, N, f, n, a, r, frac in rows:
            print(f"| {name} | {K} | {N} | {f:.3f} | {n:.3f} | {a:.3f} | {r:.3f} | {frac:.2f} |")
    dist.barrier()
    torch.cuda.synchronize()
    pc.destroy()
    return 0


if __name__ == "__main__":
    sys.exit(main())
