"""Spawn N CPU ranks (gloo) running a module-level function; failures in any rank fail the test."""
import os
import socket
import sys
import traceback

import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, err_q):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), LOCAL_WORLD_SIZE=str(world),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="1")
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        import torch

        torch.set_num_threads(1)
        fn(rank, world, *args)
    except Exception:
        err_q.put((rank, traceback.format_exc()))
        raise


def run_dist(fn, world: int, *args, timeout: float = 300):
    ctx = mp.get_context("spawn")
    err_q = ctx.SimpleQueue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, err_q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    errors = []
    while not err_q.empty():
        errors.append(err_q.get())
    for p in procs:
        if p.is_alive():
            p.kill()
            errors.append((-1, "rank timed out"))
    bad = [p.exitcode for p in procs if p.exitcode != 0]
    if errors or bad:
        msg = "\n".join(f"[rank {r}]\n{tb}" for r, tb in errors) or f"exit codes {bad}"
        raise AssertionError(msg)
