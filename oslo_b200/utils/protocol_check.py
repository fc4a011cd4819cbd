"""Exhaustive host-side check of the flag / double-buffer protocol that the fused collective kernels use.

The kernels exchange data through peer-mapped buffers that are double-buffered by the parity of a per-group call
counter (the "epoch"); flags hold the epoch of the last hand-off and are never cleared, and there is NO trailing barrier
after a call.  The safety argument is "a rank can be at most one call ahead of any peer, because finishing a call needs
data from every peer".  This module does not trust the argument: it explores EVERY interleaving of a small system
(2-3 ranks, a few calls) and checks, at every step, that

* no buffer half is overwritten while a peer still has to read, or is reading, what the previous call of the same
  parity put there (write-after-read), and
* every read returns the data of the call it belongs to (read-after-write through the flags).

A rank's call is modelled at the granularity at which other ranks can observe it:

  all-gather     W   write own ``in[parity]``
                 A   announce: ``ag_ready[peer][me] = epoch`` on every peer
                 Rt  for every peer t: wait ``ag_ready[me][t] >= epoch``, then read t's ``in[parity]`` (begin, end)
  reduce-scatter St  for every peer t: write my partial into t's ``slots[parity][me]`` (begin, end), then
                     ``rs_flag[t][me] = epoch``
                 F   wait ``rs_flag[me][t] >= epoch`` for all t, read ``slots[parity][*]`` (begin, end)

Used by ``tests/test_protocol_check.py``; ``explore`` is generic enough to model-check variations before they are
written as kernels (e.g. dropping the parity, which it rejects).
"""
from __future__ import annotations

from collections import deque
from typing import List, Sequence, Tuple


def _program(kind: str, me: int, n: int) -> List[Tuple]:
    peers = [t for t in range(n) if t != me]
    if kind == "ag":
        prog = [("write_in",), ("announce",)]
        for t in peers:
            prog += [("wait_ag", t), ("read_in_begin", t), ("read_in_end", t)]
        return prog
    if kind == "rs":
        prog = []
        for t in peers:
            prog += [("write_slot_begin", t), ("write_slot_end", t), ("flag_rs", t)]
        prog += [("wait_rs",), ("read_slots_begin",), ("read_slots_end",)]
        return prog
    raise ValueError(kind)


def explore(n_ranks: int, calls: Sequence[str], double_buffered: bool = True, max_states: int = 2_000_000):
    """Breadth-first search over all interleavings.  Returns ``(ok, states_visited, message)``."""
    n = n_ranks
    programs = [[(e + 1, step) for e, kind in enumerate(calls) for step in _program(kind, r, n)] for r in range(n)]

    def parity(epoch):
        return epoch & 1 if double_buffered else 0

    # state: (pc per rank, ag_ready[n][n], rs_flag[n][n], in_data[n][2], slot_data[n][2][n], active reads / writes)
    init = (tuple([0] * n), tuple([0] * (n * n)), tuple([0] * (n * n)), tuple([0] * (n * 2)), tuple([0] * (n * 2 * n)),
            frozenset())
    seen = {init}
    queue = deque([init])
    visited = 0
    while queue:
        state = queue.popleft()
        visited += 1
        if visited > max_states:
            return False, visited, "state space larger than max_states"
        pcs, ag, rs, ind, slot, active = state
        progressed = False
        for r in range(n):
            if pcs[r] >= len(programs[r]):
                continue
            epoch, step = programs[r][pcs[r]]
            p = parity(epoch)
            ag2, rs2, ind2, slot2, act2 = list(ag), list(rs), list(ind), list(slot), set(active)
            op = step[0]
            if op == "write_in":
                # nobody may be reading this half, and everybody who needed the previous contents must have read them
                for (kind, owner, half, reader, ep) in active:
                    if kind == "read_in" and owner == r and half == p:
                        return False, visited, f"rank {r} overwrites in[{p}] (call {epoch}) while rank {reader} reads call {ep}"
                prev = ind[r * 2 + p]
                if prev:
                    for t in range(n):
                        if t != r and not _has_read(programs[t], pcs[t], prev, r):
                            return False, visited, f"rank {r} overwrites in[{p}] of call {prev} before rank {t} read it"
                ind2[r * 2 + p] = epoch
            elif op == "announce":
                for t in range(n):
                    ag2[t * n + r] = epoch
            elif op == "wait_ag":
                if ag[r * n + step[1]] < epoch:
                    continue  # blocked
            elif op == "read_in_begin":
                t = step[1]
                if ind[t * 2 + p] != epoch:
                    return False, visited, f"rank {r} reads in[{p}] of rank {t} for call {epoch} but finds call {ind[t * 2 + p]}"
                act2.add(("read_in", t, p, r, epoch))
            elif op == "read_in_end":
                act2.discard(("read_in", step[1], p, r, epoch))
            elif op == "write_slot_begin":
                t = step[1]
                for (kind, owner, half, reader, ep) in active:
                    if kind == "read_slots" and owner == t and half == p:
                        return False, visited, f"rank {r} writes slots[{p}] of rank {t} (call {epoch}) while it reads call {ep}"
                prev = slot[(t * 2 + p) * n + r]
                if prev and not _has_reduced(programs[t], pcs[t], prev):
                    return False, visited, f"rank {r} overwrites its partial of call {prev} on rank {t} before it was reduced"
                slot2[(t * 2 + p) * n + r] = epoch
            elif op == "write_slot_end":
                pass
            elif op == "flag_rs":
                rs2[step[1] * n + r] = epoch
            elif op == "wait_rs":
                if any(rs[r * n + t] < epoch for t in range(n) if t != r):
                    continue
            elif op == "read_slots_begin":
                for t in range(n):
                    if t != r and slot[(r * 2 + p) * n + t] != epoch:
                        return False, visited, f"rank {r} reduces call {epoch} but slot of rank {t} holds call {slot[(r * 2 + p) * n + t]}"
                act2.add(("read_slots", r, p, r, epoch))
            elif op == "read_slots_end":
                act2.discard(("read_slots", r, p, r, epoch))
            progressed = True
            npcs = list(pcs)
            npcs[r] += 1
            nxt = (tuple(npcs), tuple(ag2), tuple(rs2), tuple(ind2), tuple(slot2), frozenset(act2))
            if nxt not in seen:
                seen.add(nxt)
                queue.append(nxt)
        if not progressed and any(pcs[r] < len(programs[r]) for r in range(n)):
            return False, visited, f"deadlock at program counters {pcs}"
    return True, visited, "ok"


def _has_read(program, pc, epoch, owner) -> bool:
    """Has the rank running ``program`` (now at ``pc``) finished reading ``owner``'s input of call ``epoch``?"""
    for i, (ep, step) in enumerate(program):
        if ep == epoch and step == ("read_in_end", owner):
            return pc > i
    return True  # that call does not read this owner (not an all-gather)


def _has_reduced(program, pc, epoch) -> bool:
    for i, (ep, step) in enumerate(program):
        if ep == epoch and step == ("read_slots_end",):
            return pc > i
    return True
