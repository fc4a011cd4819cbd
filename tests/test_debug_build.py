"""The debug build of the CUDA library: ``-DOSLO_DEBUG_BOUNDS`` turns OSLO_IN_BOUNDS into a check that records a status code
and skips the access; the loader picks that library when OSLO_B200_DEBUG_BOUNDS=1."""
import ctypes
from pathlib import Path

from oslo_b200.csrc import build
from oslo_b200.ops import _lib


def test_debug_flag_reaches_nvcc(monkeypatch, tmp_path):
    seen = []

    class _Done:
        returncode, stdout, stderr = 0, "", ""

    def fake_run(cmd, **kw):
        seen.append(cmd)
        out = Path(cmd[cmd.index("-o") + 1])
        out.parent.mkdir(parents=True, exist_ok=True)
        out.write_bytes(b"")
        return _Done()

    monkeypatch.setattr(build.subprocess, "run", fake_run)
    monkeypatch.setattr(build, "OBJ_DIR", tmp_path / "obj")
    monkeypatch.setattr(build, "LIB_DIR", tmp_path)
    out = build.build_cuda(debug_bounds=True)
    assert out.name == "liboslo_b200_cuda_debug.so"
    compiles = [c for c in seen if "-c" in c]
    assert compiles and all("-DOSLO_DEBUG_BOUNDS" in c for c in compiles)
    assert all("obj_debug" in c[c.index("-o") + 1] for c in compiles)
    assert all(any("compute_100a" in a for a in c) for c in compiles)
    seen.clear()
    out = build.build_cuda(debug_bounds=False)
    assert out.name == "liboslo_b200_cuda.so" and not any("-DOSLO_DEBUG_BOUNDS" in c for c in seen)


def test_loader_selects_debug_library(monkeypatch):
    opened = []
    monkeypatch.setattr(ctypes, "CDLL", lambda p: opened.append(p) or object())
    monkeypatch.setenv("OSLO_B200_AUTOBUILD", "0")
    monkeypatch.setattr(Path, "exists", lambda self: True)
    for flag, name in (("1", "liboslo_b200_cuda_debug.so"), ("0", "liboslo_b200_cuda.so")):
        monkeypatch.setenv("OSLO_B200_DEBUG_BOUNDS", flag)
        _lib._load_cuda_lib.cache_clear()
        _lib._load_cuda_lib()
        assert opened[-1].endswith(name)
    _lib._load_cuda_lib.cache_clear()


def test_checks_skip_instead_of_trapping():
    src = Path(build.CSRC)
    common = (src / "common.cuh").read_text()
    assert "#define OSLO_IN_BOUNDS(cond, status) (true)" in common and "kStatusBoundsViolation" in common
    core = (src / "gemm_core.cuh").read_text()
    assert core.count("OSLO_IN_BOUNDS(") >= 4
    for text in (common, core):
        assert "__trap" not in text and "assert(" not in text
