"""Host-side failure detection: per-rank heartbeats in the rendezvous store, and a status-word check for kernels.

* ``Heartbeat(store, rank, world)`` starts a daemon thread that bumps ``hb/{rank}`` every ``period`` seconds.
  ``stale_ranks(timeout)`` lists the ranks whose counter has not moved for ``timeout`` seconds; ``assert_alive`` raises
  ``PeerFailure`` — call it between steps, BEFORE launching the next fused kernel or collective, so a dead peer is
  learnt on the host instead of through a device-side wait running out.
* ``check_device_status()`` reads the word in which this library's kernels record a bounded wait that ran out (they
  return instead of spinning forever) and raises with the decoded reason.

The reference has no failure detection (its pipeline workers busy-wait forever: oslo/torch/nn/parallel/
pipeline_parallel/_sync.py:17-40); recovery here is "notice, stop cleanly, resume from the last checkpoint"
(``Trainer.train(resume_from_checkpoint=...)``).
"""
from __future__ import annotations

import threading
import time
from typing import List, Optional

import torch.distributed as dist


class PeerFailure(RuntimeError):
    pass


class Heartbeat:
    def __init__(self, store, rank: int, world_size: int, period: float = 0.5, prefix: str = "hb"):
        self.store, self.rank, self.world, self.period, self.prefix = store, rank, world_size, period, prefix
        self._stop = threading.Event()
        self._last = {r: (None, time.monotonic()) for r in range(world_size)}
        self._thread = threading.Thread(target=self._run, daemon=True)
        self.store.add(f"{prefix}/{rank}", 1)
        self._thread.start()

    @classmethod
    def from_context(cls, parallel_context, period: float = 0.5, port_offset: int = 17) -> "Heartbeat":
        """A dedicated TCP store next to the job's rendezvous port (the default store is busy serving collectives)."""
        rank = parallel_context.get_global_rank()
        world = dist.get_world_size()
        store = dist.TCPStore(parallel_context.host, parallel_context.port + port_offset, world, is_master=rank == 0,
                              wait_for_workers=False)
        return cls(store, rank, world, period)

    def _run(self):
        while not self._stop.wait(self.period):
            try:
                self.store.add(f"{self.prefix}/{self.rank}", 1)
            except Exception:
                return

    def stop(self):
        self._stop.set()

    def stale_ranks(self, timeout: float) -> List[int]:
        now = time.monotonic()
        out = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                cur = int(self.store.add(f"{self.prefix}/{r}", 0))
            except Exception:
                cur = None
            prev, seen = self._last[r]
            if cur is not None and cur != prev:
                self._last[r] = (cur, now)
            elif now - seen > timeout:
                out.append(r)
        return out

    def assert_alive(self, timeout: float = 5.0):
        dead = self.stale_ranks(timeout)
        if dead:
            raise PeerFailure(f"no heartbeat from rank(s) {dead} for more than {timeout} s")


def check_device_status(device=None):
    """Raise if a kernel on ``device`` gave up on a bounded wait since the last check (synchronises the device)."""
    from oslo_b200.ops import _lib

    _lib.check_status(device)
