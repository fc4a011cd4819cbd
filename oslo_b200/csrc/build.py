"""In-tree build of the native libraries.

Two shared objects are produced next to this file's package:

* ``oslo_b200/_lib/liboslo_b200_cuda.so``  every ``csrc/*.cu`` compiled by nvcc for
  ``sm_100a`` only (``-gencode arch=compute_100a,code=sm_100a``); plain
  ``extern "C"`` entry points taking raw device pointers and a stream, called from
  Python through ``ctypes`` (no libtorch dependency, so a rebuild takes seconds).
* ``oslo_b200/_lib/liboslo_b200_cpu.so``   ``csrc/cpu/*.cpp`` compiled by g++ with
  AVX-512/AVX2 + OpenMP (CPU Adam / Adagrad, memory planner, partitioner core).

Replaces the reference's per-extension JIT ``Binder`` (``oslo/torch/_C/__init__.py:249-680``).
Run as ``python -m oslo_b200.csrc.build`` or call :func:`build_all`.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
LIB_DIR = PKG / "_lib"
OBJ_DIR = LIB_DIR / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
    "--expt-relaxed-constexpr",
]
# no -march=native: SIMD bodies are selected at run time, so the library runs on any x86-64 host
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-fopenmp", "-shared"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _stamp(src: Path, flags) -> str:
    h = hashlib.sha1()
    h.update(src.read_bytes())
    for hdr in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(hdr.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def _compile_one(src: Path, verbose: bool, debug_bounds: bool = False) -> Path:
    obj_dir = OBJ_DIR.with_name("obj_debug") if debug_bounds else OBJ_DIR
    obj = obj_dir / (src.stem + ".o")
    stamp_file = obj_dir / (src.stem + ".stamp")
    flags = list(NVCC_FLAGS) + (["-DOSLO_DEBUG_BOUNDS"] if debug_bounds else [])
    if verbose:
        flags += ["-Xptxas", "-v"]
    stamp = _stamp(src, flags)
    if obj.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return obj
    cmd = [_nvcc(), *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    stamp_file.write_text(stamp)
    return obj


def build_cuda(verbose: bool = False, debug_bounds: bool = False) -> Path:
    """Compile every ``*.cu`` and link the CUDA library.  ``debug_bounds`` builds ``liboslo_b200_cuda_debug.so`` with
    ``-DOSLO_DEBUG_BOUNDS``: index checks that record a status code and skip the access (never trap); it is loaded instead
    of the normal library when ``OSLO_B200_DEBUG_BOUNDS=1``."""
    (OBJ_DIR.with_name("obj_debug") if debug_bounds else OBJ_DIR).mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    with cf.ThreadPoolExecutor(max_workers=min(8, len(sources) or 1)) as pool:
        objs = list(pool.map(lambda s: _compile_one(s, verbose, debug_bounds), sources))
    out = LIB_DIR / ("liboslo_b200_cuda_debug.so" if debug_bounds else "liboslo_b200_cuda.so")
    newest = max(o.stat().st_mtime for o in objs)
    if not out.exists() or out.stat().st_mtime < newest:
        cmd = [_nvcc(), "-shared", "-o", str(out), *map(str, objs), "-lcudart", "-Xcompiler", "-fPIC"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return out


def build_cpu() -> Path:
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    sources = sorted((CSRC / "cpu").glob("*.cpp"))
    out = LIB_DIR / "liboslo_b200_cpu.so"
    if not sources:
        return out
    newest = max(s.stat().st_mtime for s in sources + sorted((CSRC / "cpu").glob("*.h")))
    if out.exists() and out.stat().st_mtime >= newest:
        return out
    cmd = ["g++", *CXX_FLAGS, "-o", str(out), *map(str, sources)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"g++ failed:\n{res.stdout}\n{res.stderr}")
    return out


def build_all(verbose: bool = False):
    return build_cuda(verbose), build_cpu()


if __name__ == "__main__":
    if "--debug-bounds" in sys.argv:
        print(build_cuda(verbose="-v" in sys.argv, debug_bounds=True))
    else:
        print(*build_all(verbose="-v" in sys.argv), sep="\n")
