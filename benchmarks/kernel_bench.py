"""Time one native kernel on one GPU and report its fraction of the measured roofline.

    python benchmarks/kernel_bench.py gemm --m 8192 --n 8192 --k 8192
    python benchmarks/kernel_bench.py layernorm --rows 65536 --hidden 2048
    python benchmarks/kernel_bench.py all

Timing: CUDA events on the launching stream, >= 3 warm-up launches, an L2 flush (a write larger than L2) before every
timed launch unless the operands exceed L2 anyway.  Denominators come from ``MEASURED_PEAKS.json`` at the repository
root (copy bandwidth and cuBLAS bf16 throughput measured on this pool); fractions are "of measured".
The same commands, with small sizes and ``--iters 1..3``, are what the ncu captures under ``profiles/`` run.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return p["hbm_gbs"], p["bf16_tflops"], "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _flush.zero_()


def time_op(fn, iters, flush=True):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush:
            flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2]


def report(name, ms, bytes_moved=None, flops=None, extra=""):
    hbm, tf, src = peaks()
    parts = [f"{name}: {ms * 1e3:.1f} us"]
    if bytes_moved:
        gbs = bytes_moved / ms / 1e6
        parts.append(f"{gbs:.0f} GB/s = {gbs / hbm:.2f} of {src} copy bandwidth")
    if flops:
        t = flops / ms / 1e9
        parts.append(f"{t:.0f} TFLOP/s = {t / tf:.2f} of {src} cuBLAS bf16")
    print(" | ".join(parts) + (" | " + extra if extra else ""), flush=True)


def bench_gemm(a):
    from oslo_b200.ops.gemm import gemm

    x = torch.randn(a.m, a.k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(a.n, a.k, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
    A = x.t().contiguous().t() if a.a_mn else x
    B = w.t().contiguous().t() if a.b_mn else w
    ms = time_op(lambda: gemm(A, B, out=out, block_n=a.block_n, two_cta=False), a.iters)
    extra = ""
    if a.m >= 256 and a.n >= 256 and not a.block_n:
        ms_pair = time_op(lambda: gemm(A, B, out=out, two_cta=True), a.iters)
        report(f"gemm_tcgen05_2cta M{a.m} N{a.n} K{a.k} a_mn{int(a.a_mn)} b_mn{int(a.b_mn)}", ms_pair,
               flops=2.0 * a.m * a.n * a.k, extra=f"one-CTA kernel {ms * 1e3:.1f} us")
    if a.compare:
        ms2 = time_op(lambda: torch.matmul(x, w.t(), out=out), a.iters)
        extra = f"cuBLAS {ms2 * 1e3:.1f} us ({ms2 / ms:.2f}x of ours)"
    report(f"gemm_tcgen05 M{a.m} N{a.n} K{a.k} a_mn{int(a.a_mn)} b_mn{int(a.b_mn)}", ms, flops=2.0 * a.m * a.n * a.k, extra=extra)


def bench_layernorm(a):
    from oslo_b200.ops.norm import layer_norm

    x = torch.randn(a.rows, a.hidden, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.ones(a.hidden, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    b = torch.zeros(a.hidden, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    n = x.numel() * 2
    ms = time_op(lambda: layer_norm(x.detach(), a.hidden, w.detach(), b.detach(), 1e-5), a.iters)
    report(f"layernorm_fwd rows{a.rows} H{a.hidden}", ms, bytes_moved=2 * n)
    y = layer_norm(x, a.hidden, w, b, 1e-5)
    g = torch.randn_like(y)
    ms = time_op(lambda: torch.autograd.grad(y, (x, w, b), g, retain_graph=True), a.iters)
    report(f"layernorm_bwd rows{a.rows} H{a.hidden}", ms, bytes_moved=3 * n)


def bench_softmax(a):
    from oslo_b200.ops.softmax import softmax_inplace_

    x = torch.randn(a.batch, a.seq, a.seq, device="cuda", dtype=torch.bfloat16)
    ms = time_op(lambda: softmax_inplace_(x, 0.125, True), a.iters)
    report(f"softmax_causal B{a.batch} S{a.seq}", ms, bytes_moved=x.numel() * 2 * 1.5, extra="bytes = causal half read + full write")


def bench_bias_gelu(a):
    from oslo_b200.ops.activation import bias_gelu

    x = torch.randn(a.rows, a.hidden, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(a.hidden, device="cuda", dtype=torch.bfloat16)
    ms = time_op(lambda: bias_gelu(x, b), a.iters)
    report(f"bias_gelu rows{a.rows} H{a.hidden}", ms, bytes_moved=2 * x.numel() * 2)


def bench_adam(a):
    from oslo_b200.optim import FusedAdam

    p = torch.randn(a.numel, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    p.grad = torch.randn_like(p)
    opt = FusedAdam([p], lr=1e-3, master_weights=True)
    ms = time_op(opt.step, a.iters)
    report(f"adamw_multi_tensor n{a.numel}", ms, bytes_moved=a.numel * (2 + 2 + 3 * 4 + 3 * 4 + 2))


def bench_ce(a):
    from oslo_b200.ops.loss import vocab_parallel_cross_entropy

    logits = torch.randn(a.rows, a.vocab, device="cuda", dtype=torch.bfloat16)
    tgt = torch.randint(0, a.vocab, (a.rows,), device="cuda")
    ms = time_op(lambda: vocab_parallel_cross_entropy(logits.clone(), tgt), a.iters)
    ms0 = time_op(lambda: logits.clone(), a.iters)
    report(f"cross_entropy rows{a.rows} V{a.vocab}", ms - ms0, bytes_moved=logits.numel() * 2 * 3, extra="stats pass + gradient pass (clone time subtracted)")


def bench_attention(a):
    from oslo_b200.ops.attention import qkv_attention

    h = a.heads * a.head_dim
    qkv = torch.randn(a.batch, a.seq, 3 * h, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    fl = 4.0 * a.batch * a.heads * a.seq * a.seq * a.head_dim / 2  # causal
    ms = time_op(lambda: qkv_attention(qkv.detach(), a.heads, a.head_dim, "h3d", True), a.iters)
    report(f"attention_fwd B{a.batch} S{a.seq} H{a.heads}x{a.head_dim}", ms, flops=fl)
    if a.seq % 256 == 0:
        import math

        from oslo_b200.ops.attention import flash_attention_forward

        q5 = qkv.detach().view(a.batch, a.seq, a.heads, 3, a.head_dim)
        q, k, v = q5[..., 0, :], q5[..., 1, :], q5[..., 2, :]
        for pp in (False, True):
            ms = time_op(lambda: flash_attention_forward(q, k, v, True, 1.0 / math.sqrt(a.head_dim), pingpong=pp), a.iters)
            report(f"attention_fwd kernel only ({'one-pass ping-pong' if pp else 'two-pass'}) B{a.batch} S{a.seq} "
                   f"H{a.heads}x{a.head_dim}", ms, flops=fl)
    out = qkv_attention(qkv, a.heads, a.head_dim, "h3d", True)
    g = torch.randn_like(out)
    from oslo_b200.ops.attention import set_backward_groups

    for groups, dq in ((1, 1), (2, 1), (2, 2)):
        set_backward_groups(groups, dq_groups=dq)
        ms = time_op(lambda: torch.autograd.grad(out, qkv, g, retain_graph=True), a.iters)
        report(f"attention_bwd (element-wise groups: {groups} in dK/dV, {dq} in dQ) B{a.batch} S{a.seq} "
               f"H{a.heads}x{a.head_dim}", ms, flops=2.5 * fl)
    set_backward_groups(2, dq_groups=1)  # the defaults


KERNELS = {"gemm": bench_gemm, "layernorm": bench_layernorm, "softmax": bench_softmax, "bias_gelu": bench_bias_gelu,
           "adam": bench_adam, "ce": bench_ce, "attention": bench_attention}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=sorted(KERNELS) + ["all"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--a-mn", action="store_true")
    ap.add_argument("--b-mn", action="store_true")
    ap.add_argument("--block-n", type=int, default=0)
    ap.add_argument("--compare", action="store_true", help="also time torch.matmul (cuBLAS)")
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--vocab", type=int, default=50304)
    ap.add_argument("--numel", type=int, default=256 * 1024 * 1024)
    a = ap.parse_args()
    from oslo_b200.ops import _lib

    if a.kernel == "all":
        a.compare = True
        for shape in [(8192, 8192, 8192), (16384, 6144, 2048), (16384, 8192, 2048), (16384, 2048, 8192)]:
            a.m, a.n, a.k = shape
            bench_gemm(a)
        a.m, a.n, a.k, a.a_mn, a.b_mn = 8192, 2048, 16384, True, True
        bench_gemm(a)
        a.a_mn = a.b_mn = False
        a.rows = 65536
        for name in ("layernorm", "bias_gelu", "softmax", "adam", "ce", "attention"):
            if name == "ce":
                a.rows = 16384
            if name == "attention":
                a.batch = 8
            KERNELS[name](a)
    else:
        KERNELS[a.kernel](a)
    torch.cuda.synchronize()
    _lib.check_status()


if __name__ == "__main__":
    main()
