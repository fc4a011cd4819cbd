"""The allocation-free column sum, called through its exported C symbol, against the ordinary entry point.

Some hosts of the kernel library cannot allocate device memory when they call it (inside a stream capture or a
stream callback, or C/C++ programs without PyTorch's allocator); ``oslo_colsum_noalloc`` serves them by keeping
its partial sums in an array built into the library.  This file checks that it gives the same column sums as
``oslo_colsum`` (which takes a caller-allocated scratch buffer) on two consecutive calls that share the built-in
array, and that it refuses an input wider than that array.  It is named to be collected last.
"""
import ctypes
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = Path(__file__).resolve().parent.parent / "oslo_b200" / "_lib" / "liboslo_b200_cuda.so"
DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _lib():
    lib = ctypes.CDLL(str(LIB))
    lib.oslo_colsum_noalloc.restype = ctypes.c_int
    lib.oslo_colsum_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                                        ctypes.c_void_p]
    lib.oslo_colsum_noalloc_max_scratch_floats.restype = ctypes.c_longlong
    lib.oslo_colsum.restype = ctypes.c_int
    lib.oslo_colsum_parts.restype = ctypes.c_int
    return lib


def _ordinary(lib, x):
    rows, h = x.shape
    sms = torch.cuda.get_device_properties(x.device).multi_processor_count
    parts = lib.oslo_colsum_parts(ctypes.c_longlong(rows), ctypes.c_int(sms))
    scratch = torch.empty(parts * h, dtype=torch.float32, device=x.device)
    out = torch.empty(h, dtype=x.dtype, device=x.device)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.oslo_colsum(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(scratch.data_ptr()),
                         ctypes.c_longlong(rows), ctypes.c_int(h), ctypes.c_int(DT[x.dtype]), ctypes.c_int(sms), stream)
    assert rc == 0
    return out


def _noalloc(lib, x):
    rows, h = x.shape
    out = torch.empty(h, dtype=x.dtype, device=x.device)  # the caller still owns input and output
    rc = lib.oslo_colsum_noalloc(x.data_ptr(), out.data_ptr(), rows, h, DT[x.dtype],
                                 torch.cuda.current_stream().cuda_stream)
    assert rc == 0, rc
    return out


def test_noalloc_colsum_matches_ordinary_entry_point_twice():
    lib = _lib()
    torch.manual_seed(0)
    # two calls in a row with different shapes and dtypes: the second reuses (and must overwrite) the built-in array
    # the third case is wide enough that (row partitions x columns) exceeds the built-in array, so the entry point has to
    # fall back to fewer partitions than the ordinary one uses
    limit = lib.oslo_colsum_noalloc_max_scratch_floats()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    wide = (20000, 65536, torch.bfloat16)
    assert lib.oslo_colsum_parts(ctypes.c_longlong(wide[0]), ctypes.c_int(sms)) * wide[1] > limit
    for rows, h, dtype in [(5000, 2048, torch.bfloat16), (777, 4096, torch.float32), wide]:
        x = torch.randn(rows, h, device="cuda", dtype=dtype)
        got = _noalloc(lib, x)
        want = _ordinary(lib, x)
        ref = x.float().sum(0)
        torch.cuda.synchronize()
        scale = ref.abs().max().item() + 1e-6
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        assert (got.float() - want.float()).abs().max().item() / scale < tol
        assert (got.float() - ref).abs().max().item() / scale < tol


def test_noalloc_colsum_refuses_misaligned_pointers_before_launching():
    lib = _lib()
    buf = torch.zeros(64 * 1024 + 64, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(1024 + 64, device="cuda", dtype=torch.bfloat16)
    stream = torch.cuda.current_stream().cuda_stream
    # an input that starts 2 bytes into an aligned buffer, then an output that does: both are refused with the argument code
    assert lib.oslo_colsum_noalloc(buf.data_ptr() + 2, out.data_ptr(), 64, 1024, 2, stream) == -1
    assert lib.oslo_colsum_noalloc(buf.data_ptr(), out.data_ptr() + 2, 64, 1024, 2, stream) == -1
    assert lib.oslo_colsum_noalloc(buf.data_ptr(), out.data_ptr(), 64, 1024, 2, stream) == 0
    torch.cuda.synchronize()
    assert float(out[:1024].float().abs().max()) == 0.0


def test_noalloc_colsum_rejects_inputs_beyond_the_builtin_scratch():
    lib = _lib()
    limit = lib.oslo_colsum_noalloc_max_scratch_floats()
    x = torch.zeros(1, limit + 8, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(limit + 8, device="cuda", dtype=torch.bfloat16)
    rc = lib.oslo_colsum_noalloc(x.data_ptr(), out.data_ptr(), 1, limit + 8, 2, torch.cuda.current_stream().cuda_stream)
    assert rc == -10
