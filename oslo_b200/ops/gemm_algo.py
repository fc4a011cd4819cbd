"""Per-shape kernel selection for the tcgen05 GEMM: an offline search that times every variant on the device and a map
that :func:`oslo_b200.ops.gemm.gemm` consults.

Counterpart of the reference's offline cuBLAS algorithm search (oslo/lightseq2/csrc/kernels/cuda/gemm_test.cpp writes a
per-shape table, cublas_algo_map.cpp loads it and the wrappers look the algorithm up at run time).  Here the "algorithms" are
this package's own kernel variants:

* ``two_cta``: the cluster kernel in which an SM pair shares a 256 x 256 tile, or the one-CTA kernel;
* ``block_n``: the one-CTA kernel's tile width (64, 128 or 256; 0 = its built-in choice).

``python -m oslo_b200.ops.gemm_algo --shapes 16384x2048x2048 16384x8192x2048 --out gemm_algo.json`` runs the search (CUDA
events, warm-up, an L2 flush between timed launches, every variant's result checked against the first) and writes the map;
``OSLO_B200_GEMM_ALGO_MAP=gemm_algo.json`` (or :func:`load`) makes ``gemm`` use it for calls that leave the choice open.
Shapes that are not in the map keep the built-in heuristic; ``M`` (the token dimension, which varies with the batch) is
matched by power-of-two bucket, ``N`` / ``K`` / operand majors / dtype exactly.
"""
from __future__ import annotations

import argparse
import json
import os
from dataclasses import asdict, dataclass
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch


@dataclass(frozen=True)
class Algo:
    two_cta: bool = False
    block_n: int = 0

    def label(self) -> str:
        return "2cta-256x256" if self.two_cta else (f"1cta-128x{self.block_n}" if self.block_n else "1cta-auto")


def m_bucket(m: int) -> int:
    """Smallest power of two >= m (so one entry serves every batch size that fills the same number of tile rows)."""
    return 1 << max(0, int(m) - 1).bit_length()


def shape_key(m: int, n: int, k: int, a_mn: int = 0, b_mn: int = 0, dtype: str = "bf16", batch: int = 1) -> str:
    return f"{m_bucket(m)}x{n}x{k}:{'t' if a_mn else 'n'}{'t' if b_mn else 'n'}:{dtype}:b{batch}"


def candidates(m: int, n: int, k: int) -> List[Algo]:
    """Variants that can run this shape: the tile must not be wider than the (8-padded) output, the cluster kernel needs
    one full 256 x 256 tile and K of at least one pipeline's depth."""
    out = [Algo(False, 0)]
    for bn in (64, 128, 256):
        if n >= bn:
            out.append(Algo(False, bn))
    if m >= 256 and n >= 256 and k >= 256:
        out.append(Algo(True, 0))
    return out


class AlgoMap:
    """``shape key -> {algo, tflops, all timings}``; JSON on disk."""

    VERSION = 1

    def __init__(self, entries: Optional[Dict[str, dict]] = None, device: str = ""):
        self.entries: Dict[str, dict] = dict(entries or {})
        self.device = device

    def set(self, key: str, algo: Algo, ms: float, flops: float, timings: Optional[Dict[str, float]] = None):
        self.entries[key] = {"algo": asdict(algo), "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12 if ms > 0 else 0.0,
                             "timings_ms": dict(timings or {})}

    def get(self, m: int, n: int, k: int, a_mn: int = 0, b_mn: int = 0, dtype: str = "bf16", batch: int = 1) -> Optional[Algo]:
        e = self.entries.get(shape_key(m, n, k, a_mn, b_mn, dtype, batch))
        if e is None:
            return None
        algo = Algo(**e["algo"])
        if algo.two_cta and (m < 256 or n < 256):
            return None  # the bucket's winner cannot run this smaller member of the bucket
        return algo

    def save(self, path: str) -> None:
        tmp = path + ".tmp"
        with open(tmp, "w") as f:
            json.dump({"version": self.VERSION, "device": self.device, "entries": self.entries}, f, indent=1, sort_keys=True)
        os.replace(tmp, path)

    @classmethod
    def load(cls, path: str) -> "AlgoMap":
        with open(path) as f:
            raw = json.load(f)
        if raw.get("version") != cls.VERSION:
            raise ValueError(f"{path}: algorithm map version {raw.get('version')} (this build reads {cls.VERSION})")
        for key, e in raw["entries"].items():
            Algo(**e["algo"])  # validates the field names
        return cls(raw["entries"], raw.get("device", ""))

    def __len__(self):
        return len(self.entries)


_ACTIVE: Optional[AlgoMap] = None
_ENV_CHECKED = False


def load(path: Optional[str]) -> Optional[AlgoMap]:
    """Make ``gemm`` consult the map at ``path`` (``None`` switches the lookup off)."""
    global _ACTIVE, _ENV_CHECKED
    _ENV_CHECKED = True
    _ACTIVE = AlgoMap.load(path) if path else None
    return _ACTIVE


def active() -> Optional[AlgoMap]:
    global _ENV_CHECKED
    if not _ENV_CHECKED:
        _ENV_CHECKED = True
        path = os.environ.get("OSLO_B200_GEMM_ALGO_MAP")
        if path:
            load(path)
    return _ACTIVE


def lookup(m: int, n: int, k: int, a_mn: int, b_mn: int, dtype: torch.dtype, batch: int) -> Optional[Algo]:
    amap = active()
    if amap is None:
        return None
    return amap.get(m, n, k, a_mn, b_mn, "bf16" if dtype == torch.bfloat16 else "fp16", batch)


def _device_timer(fn: Callable[[], None], warmup: int, iters: int, flush: Optional[torch.Tensor]) -> float:
    """Median milliseconds of ``fn`` with CUDA events on the current stream; ``flush`` (a buffer larger than L2) is
    rewritten before every timed launch so that no variant is measured on operands the previous one left in cache."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        stop.record()
        stop.synchronize()
        times.append(start.elapsed_time(stop))
    times.sort()
    return times[len(times) // 2]


def search(shapes: Iterable[Tuple[int, int, int]], dtype: torch.dtype = torch.bfloat16, a_mn: int = 0, b_mn: int = 0,
           warmup: int = 3, iters: int = 10, amap: Optional[AlgoMap] = None,
           run: Optional[Callable[[int, int, int, Algo], Callable[[], torch.Tensor]]] = None,
           timer: Optional[Callable[[Callable[[], None]], float]] = None, log: Callable[[str], None] = print) -> AlgoMap:
    """Time every candidate of every ``(M, N, K)`` and record the fastest whose result agrees with the first candidate's.

    ``run(m, n, k, algo)`` returns a closure that launches the product and returns its output (default: random operands
    on the current CUDA device through :func:`oslo_b200.ops.gemm.gemm`); ``timer(closure)`` returns milliseconds
    (default: CUDA events, median of ``iters`` after ``warmup``, L2 flushed between launches).  Both can be replaced,
    which is how the selection logic is tested without a device."""
    amap = amap if amap is not None else AlgoMap(device=torch.cuda.get_device_name() if torch.cuda.is_available() else "")
    flush = None
    if timer is None:
        flush = torch.empty(160 << 20, dtype=torch.uint8, device="cuda")
        timer = lambda fn: _device_timer(fn, warmup, iters, flush)  # noqa: E731
    if run is None:
        run = _default_runner(dtype, a_mn, b_mn)
    name = "bf16" if dtype == torch.bfloat16 else "fp16"
    for m, n, k in shapes:
        best: Optional[Tuple[float, Algo]] = None
        timings: Dict[str, float] = {}
        reference = None
        for algo in candidates(m, n, k):
            try:
                fn = run(m, n, k, algo)
                out = fn()
            except RuntimeError as e:  # a variant that refuses the shape is skipped, not fatal
                log(f"  {m}x{n}x{k} {algo.label()}: refused ({str(e)[:80]})")
                continue
            if reference is None:
                reference = out.float() if torch.is_tensor(out) else out
            elif torch.is_tensor(out):
                err = (out.float() - reference).abs().max().item()
                scale = reference.abs().max().item() + 1e-6
                if err > 2e-2 * scale:
                    log(f"  {m}x{n}x{k} {algo.label()}: result differs by {err:.3g} (scale {scale:.3g}), skipped")
                    continue
            ms = float(timer(fn))
            timings[algo.label()] = ms
            if best is None or ms < best[0]:
                best = (ms, algo)
        if best is None:
            log(f"{m}x{n}x{k}: no variant ran")
            continue
        amap.set(shape_key(m, n, k, a_mn, b_mn, name), best[1], best[0], 2.0 * m * n * k, timings)
        log(f"{m}x{n}x{k}: {best[1].label()} {best[0]:.4f} ms = {2.0 * m * n * k / best[0] / 1e9:.1f} TFLOP/s  "
            + " ".join(f"{k_}={v:.4f}" for k_, v in sorted(timings.items())))
    return amap


def _default_runner(dtype, a_mn, b_mn):
    from .gemm import gemm

    def make(m, n, k, algo: Algo):
        g = torch.Generator(device="cuda").manual_seed(m * 31 + n * 17 + k)
        a = torch.randn((k, m) if a_mn else (m, k), device="cuda", dtype=dtype, generator=g)
        b = torch.randn((k, n) if b_mn else (n, k), device="cuda", dtype=dtype, generator=g)
        a_op, b_op = (a.t() if a_mn else a), (b.t() if b_mn else b)
        out = torch.empty(m, n, device="cuda", dtype=dtype)
        return lambda: gemm(a_op, b_op, out=out, two_cta=algo.two_cta, block_n=algo.block_n)

    return make


def parse_shapes(items: Sequence[str]) -> List[Tuple[int, int, int]]:
    shapes = []
    for it in items:
        parts = it.lower().replace(",", "x").split("x")
        if len(parts) != 3:
            raise ValueError(f"shape {it!r} is not MxNxK")
        shapes.append(tuple(int(p) for p in parts))
    return shapes


def model_shapes(hidden: int, ffn: int, tokens: int, vocab: int = 0, tp: int = 1) -> List[Tuple[int, int, int]]:
    """The forward products of one transformer layer (and the head) under 1-D tensor parallelism of size ``tp``; the two
    backward products of each are searched by passing the transposed majors on a second / third run."""
    s = [(tokens, 3 * hidden // tp, hidden), (tokens, hidden, hidden // tp), (tokens, ffn // tp, hidden), (tokens, hidden, ffn // tp)]
    if vocab:
        s.append((tokens, vocab // tp, hidden))
    return s


def main(argv=None):
    ap = argparse.ArgumentParser(description="offline per-shape search over the tcgen05 GEMM variants")
    ap.add_argument("--shapes", nargs="*", default=[], help="MxNxK ...")
    ap.add_argument("--model", nargs=3, type=int, metavar=("HIDDEN", "FFN", "TOKENS"), help="search a transformer layer's products")
    ap.add_argument("--vocab", type=int, default=0)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--backward", action="store_true", help="also search the dX (b transposed) and dW (a, b transposed) forms")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", default="gemm_algo.json")
    args = ap.parse_args(argv)
    shapes = parse_shapes(args.shapes)
    if args.model:
        shapes += model_shapes(args.model[0], args.model[1], args.model[2], args.vocab, args.tp)
    if not shapes:
        ap.error("give --shapes or --model")
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    amap = AlgoMap.load(args.out) if os.path.exists(args.out) else None
    amap = search(shapes, dtype, iters=args.iters, amap=amap)
    if args.backward:
        # y = x W^T: dX = dY W has W as the MN-major b operand; dW = dY^T X has both operands MN-major
        search([(m, k, n) for m, n, k in shapes], dtype, 0, 1, iters=args.iters, amap=amap)
        search([(n, k, m) for m, n, k in shapes], dtype, 1, 1, iters=args.iters, amap=amap)
    amap.save(args.out)
    print(f"wrote {len(amap)} entries to {args.out}")


if __name__ == "__main__":
    main()
