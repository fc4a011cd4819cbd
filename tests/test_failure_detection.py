"""Failure detection without faulting a GPU: a peer that stops heart-beating is noticed on the host, a collective whose
peer never joins ends with an error after the process-group timeout, and (on a GPU) a wait on a flag that nothing sets
runs out, records a status and leaves the context usable."""
import ctypes
import os
import time

import pytest
import torch

from dist_utils import run_dist


def _heartbeat_worker(rank, world):
    import torch.distributed as dist

    from oslo_b200 import ParallelContext
    from oslo_b200.utils.watchdog import Heartbeat, PeerFailure

    pc = ParallelContext.from_torch(data_parallel_size=world, backend="gloo")
    hb = Heartbeat.from_context(pc, period=0.1)
    dist.barrier()
    time.sleep(0.5)
    assert hb.stale_ranks(timeout=1.0) == []
    dist.barrier()
    if rank == 1:
        hb.stop()  # rank 1 "dies" between steps: its heartbeat stops, it makes no further collective call
        time.sleep(3.0)
        return
    deadline = time.time() + 5
    noticed = False
    while time.time() < deadline:
        try:
            hb.assert_alive(timeout=1.0)
        except PeerFailure as e:
            noticed = "rank(s) [1]" in str(e)
            break
        time.sleep(0.2)
    assert noticed, "the stopped heartbeat was not noticed"


def test_stopped_heartbeat_is_noticed_on_the_host():
    run_dist(_heartbeat_worker, 2, timeout=120)


def _timeout_worker(rank, world):
    import torch.distributed as dist

    from oslo_b200 import ParallelContext

    pc = ParallelContext.from_torch(data_parallel_size=world, backend="gloo", timeout_s=3)
    dist.barrier()
    if rank == 1:
        time.sleep(8)  # never joins the next collective in time
        return
    t0 = time.time()
    with pytest.raises(Exception):
        dist.all_reduce(torch.ones(4))
    assert time.time() - t0 < 7.5, "the collective did not give up within the process-group timeout"


def test_collective_with_absent_peer_errors_after_timeout():
    run_dist(_timeout_worker, 2, timeout=120)


@pytest.mark.gpu
def test_device_wait_runs_out_and_reports_status():
    from oslo_b200.ops import _lib
    from oslo_b200.ops.gemm import gemm

    dev = torch.device("cuda", 0)
    lib = _lib.cuda_lib()
    flags = torch.zeros(64, dtype=torch.int32, device=dev)
    status = _lib.status_word(dev)
    status.zero_()
    # a "group" of two ranks whose second member never shows up: rank 0 signals itself only and waits for slot 1
    peers = (ctypes.c_void_p * 2)(flags.data_ptr(), flags.data_ptr())
    t0 = time.time()
    rc = lib.oslo_symm_barrier(peers, ctypes.c_void_p(flags.data_ptr()), ctypes.c_int(0), ctypes.c_int(2), ctypes.c_int(1),
                               ctypes.c_void_p(status.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), None)
    assert rc == 0
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert 1.0 < waited < 10.0, waited  # the wait is bounded (about two seconds)
    with pytest.raises(RuntimeError, match="peer flag"):
        _lib.check_status(dev)
    # the context is still usable afterwards
    a = torch.randn(128, 64, device=dev, dtype=torch.bfloat16)
    b = torch.randn(64, 64, device=dev, dtype=torch.bfloat16)
    y = gemm(a, b)
    torch.cuda.synchronize()
    _lib.check_status(dev)
    assert torch.isfinite(y.float()).all()
