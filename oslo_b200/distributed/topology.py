"""Pure-Python rank topology: which global ranks form which group in each mode.

Nothing here touches ``torch.distributed``; the functions return plain lists so
the formulas can be unit-tested for any world size on a laptop.  The runtime
(`parallel_context.py`) turns the lists into process groups, creating each
distinct rank list exactly once.

Rank formulas follow the reference initializers
(``oslo/torch/distributed/_initializers/*.py``):

* DATA      ``i + j * (world / dp)``                     (initializer_data.py:22-27)
* MODEL     contiguous blocks of ``world / dp``          (initializer_model.py:25-29)
* TENSOR    contiguous blocks of ``tp``                  (initializer_tensor.py:22-26)
* PIPELINE  stride ``world / dp / pp`` inside a DP block (initializer_pipeline.py:17-25)
* SEQUENCE  contiguous blocks of ``sp``; SEQUENCE_DP blocks of ``world / pp``
                                                         (initializer_sequence.py:24-28,67-68)
* EXPERT    consecutive ``ep`` slices of ``range(i, world, tp)``
                                                         (initializer_expert.py:76-101)
* 2D        ROW ``base + j*q + k``, COL ``base + j + k*q``
                                                         (initializer_tensor_2d.py:42-45,101-104)
* 2.5D      rank ``base + i + q*(j + q*k)``; ROW varies i, COL j, DEP k, XZ (k, j)
                                                         (initializer_tensor_2p5d.py:48-250)
* 3D        rank ``base + i + c*(j + c*k)``; INPUT varies j, WEIGHT i, OUTPUT k
                                                         (initializer_tensor_3d.py:36-135)
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional

from .parallel_mode import ParallelMode

Groups = List[List[int]]


def _isqrt_exact(n: int, what: str) -> int:
    q = math.isqrt(n)
    if q * q != n:
        raise ValueError(f"{what}: {n} is not a perfect square")
    return q


def _icbrt_exact(n: int, what: str) -> int:
    c = round(n ** (1.0 / 3.0))
    if c ** 3 != n:
        raise ValueError(f"{what}: {n} is not a perfect cube")
    return c


@dataclass(frozen=True)
class Topology:
    """Sizes of every parallel dimension of one job."""

    world_size: int
    data_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    tensor_parallel_size: int = 1
    sequence_parallel_size: int = 1
    expert_parallel_size: int = 1
    tensor_parallel_mode: Optional[ParallelMode] = ParallelMode.TENSOR_1D
    tensor_parallel_depth: Optional[int] = None
    #: True when the expert group overlays the data group (EP ⊆ DP on the same
    #: ranks, e.g. EP=8 and DP=8 on 8 GPUs).  The reference can only express
    #: ``world == dp*pp*tp*sp*ep`` (parallel_context.py:437-450); both are accepted.
    expert_overlay: bool = False

    # ------------------------------------------------------------------ checks
    def validate(self) -> "Topology":
        w, dp, pp, tp, sp, ep = (
            self.world_size,
            self.data_parallel_size,
            self.pipeline_parallel_size,
            self.tensor_parallel_size,
            self.sequence_parallel_size,
            self.expert_parallel_size,
        )
        for name, v in (("data", dp), ("pipeline", pp), ("tensor", tp), ("sequence", sp), ("expert", ep)):
            if not isinstance(v, int) or v < 1:
                raise ValueError(f"{name}_parallel_size must be a positive int, got {v!r}")
        if sp > 1 and tp > 1:
            raise ValueError(
                "sequence (ring) parallelism and tensor parallelism are mutually exclusive: "
                f"sequence_parallel_size={sp}, tensor_parallel_size={tp}"
            )
        if tp > 1 and self.tensor_parallel_mode is None:
            raise ValueError("tensor_parallel_mode must be given when tensor_parallel_size > 1")
        mode = self.tensor_parallel_mode
        if mode is not None and mode not in (
            ParallelMode.TENSOR_1D,
            ParallelMode.TENSOR_2D,
            ParallelMode.TENSOR_2P5D,
            ParallelMode.TENSOR_3D,
        ):
            raise ValueError(f"unsupported tensor_parallel_mode {mode}")
        if mode == ParallelMode.TENSOR_2D:
            _isqrt_exact(tp, "2D tensor parallel size")
        if mode == ParallelMode.TENSOR_2P5D:
            d = self.tensor_parallel_depth
            if d is None:
                raise ValueError("tensor_parallel_depth is required for 2.5D tensor parallelism")
            if tp % d:
                raise ValueError(f"2.5D: tensor size {tp} not divisible by depth {d}")
            _isqrt_exact(tp // d, "2.5D tensor parallel size / depth")
        if mode == ParallelMode.TENSOR_3D:
            _icbrt_exact(tp, "3D tensor parallel size")
        base = dp * pp * tp * sp
        if self.expert_overlay:
            if w != base:
                raise ValueError(f"world size {w} != dp*pp*tp*sp = {base}")
            if dp % ep:
                raise ValueError(f"expert overlay needs expert size {ep} to divide data size {dp}")
        elif w != base * ep:
            raise ValueError(
                f"world size {w} != data ({dp}) * pipeline ({pp}) * tensor ({tp}) * sequence ({sp}) * expert ({ep})"
            )
        return self

    # ------------------------------------------------------------- group lists
    def groups(self, mode: ParallelMode) -> Groups:
        """All groups (lists of global ranks) that exist in ``mode``."""
        w, dp, pp, tp, sp, ep = (
            self.world_size,
            self.data_parallel_size,
            self.pipeline_parallel_size,
            self.tensor_parallel_size,
            self.sequence_parallel_size,
            self.expert_parallel_size,
        )
        M = ParallelMode
        if mode == M.GLOBAL:
            return [list(range(w))]
        if mode == M.DATA:
            n = w // dp
            return [[i + j * n for j in range(dp)] for i in range(n)]
        if mode == M.MODEL:
            n = w // dp
            return [list(range(i * n, (i + 1) * n)) for i in range(dp)]
        if mode in (M.TENSOR, M.TENSOR_1D, M.TENSOR_2D, M.TENSOR_2P5D, M.TENSOR_3D):
            return [list(range(i * tp, (i + 1) * tp)) for i in range(w // tp)]
        if mode == M.PIPELINE:
            block = w // dp
            stride = block // pp
            return [
                [d * block + i + s * stride for s in range(pp)]
                for d in range(dp)
                for i in range(stride)
            ]
        if mode == M.SEQUENCE:
            return [list(range(i * sp, (i + 1) * sp)) for i in range(w // sp)]
        if mode == M.SEQUENCE_DP:
            n = w // pp
            return [list(range(i * n, (i + 1) * n)) for i in range(pp)]
        if mode == M.EXPERT:
            return self.expert_groups(ep)
        if mode in (M.TENSOR_2D_ROW, M.TENSOR_2D_COL):
            q = _isqrt_exact(tp, "2D tensor parallel size")
            out = []
            for base in range(0, w, tp):
                for j in range(q):
                    if mode == M.TENSOR_2D_ROW:
                        out.append([base + j * q + k for k in range(q)])
                    else:
                        out.append([base + j + k * q for k in range(q)])
            return out
        if mode in (M.TENSOR_2P5D_ROW, M.TENSOR_2P5D_COL, M.TENSOR_2P5D_DEP, M.TENSOR_2P5D_XZ):
            d = self.tensor_parallel_depth
            q = _isqrt_exact(tp // d, "2.5D tensor parallel size / depth")
            out = []
            for base in range(0, w, tp):
                if mode == M.TENSOR_2P5D_ROW:
                    for k in range(d):
                        for j in range(q):
                            out.append([base + i + q * (j + q * k) for i in range(q)])
                elif mode == M.TENSOR_2P5D_COL:
                    for k in range(d):
                        for i in range(q):
                            out.append([base + i + q * (j + q * k) for j in range(q)])
                elif mode == M.TENSOR_2P5D_DEP:
                    for j in range(q):
                        for i in range(q):
                            out.append([base + i + q * (j + q * k) for k in range(d)])
                else:
                    for i in range(q):
                        out.append([base + i + q * (j + q * k) for k in range(d) for j in range(q)])
            return out
        if mode in (M.TENSOR_3D_INPUT, M.TENSOR_3D_WEIGHT, M.TENSOR_3D_OUTPUT):
            c = _icbrt_exact(tp, "3D tensor parallel size")
            out = []
            for base in range(0, w, tp):
                if mode == M.TENSOR_3D_INPUT:
                    for i in range(c):
                        for k in range(c):
                            out.append([base + i + c * (j + c * k) for j in range(c)])
                elif mode == M.TENSOR_3D_WEIGHT:
                    for j in range(c):
                        for k in range(c):
                            out.append([base + i + c * (j + c * k) for i in range(c)])
                else:
                    for i in range(c):
                        for j in range(c):
                            out.append([base + i + c * (j + c * k) for k in range(c)])
            return out
        raise KeyError(mode)

    def expert_groups(self, ep: int) -> Groups:
        """Expert groups of size ``ep`` (also used per layer for "pyramid" MoE)."""
        w, tp = self.world_size, self.tensor_parallel_size
        out = []
        for i in range(tp):
            strided = list(range(i, w, tp))
            for s in range(0, len(strided), ep):
                chunk = strided[s : s + ep]
                if len(chunk) == ep:
                    out.append(chunk)
        return out

    def active_modes(self) -> List[ParallelMode]:
        """Modes for which groups are created, in creation order."""
        M = ParallelMode
        modes = [M.GLOBAL, M.DATA, M.MODEL, M.TENSOR, M.PIPELINE, M.SEQUENCE, M.SEQUENCE_DP, M.EXPERT]
        tpm = self.tensor_parallel_mode
        if tpm == M.TENSOR_1D:
            modes += [M.TENSOR_1D]
        elif tpm == M.TENSOR_2D:
            modes += [M.TENSOR_2D, M.TENSOR_2D_ROW, M.TENSOR_2D_COL]
        elif tpm == M.TENSOR_2P5D:
            modes += [M.TENSOR_2P5D, M.TENSOR_2P5D_ROW, M.TENSOR_2P5D_COL, M.TENSOR_2P5D_DEP, M.TENSOR_2P5D_XZ]
        elif tpm == M.TENSOR_3D:
            modes += [M.TENSOR_3D, M.TENSOR_3D_INPUT, M.TENSOR_3D_WEIGHT, M.TENSOR_3D_OUTPUT]
        return modes

    def group_of(self, mode: ParallelMode, rank: int) -> List[int]:
        for g in self.groups(mode):
            if rank in g:
                return g
        raise ValueError(f"rank {rank} is in no {mode} group")

    def membership(self, rank: int) -> Dict[ParallelMode, List[int]]:
        return {m: self.group_of(m, rank) for m in self.active_modes()}

    # convenience: summa / cubic dims
    @property
    def summa_dim(self) -> int:
        if self.tensor_parallel_mode == ParallelMode.TENSOR_2D:
            return _isqrt_exact(self.tensor_parallel_size, "2D")
        if self.tensor_parallel_mode == ParallelMode.TENSOR_2P5D:
            return _isqrt_exact(self.tensor_parallel_size // self.tensor_parallel_depth, "2.5D")
        raise ValueError("summa_dim is defined for 2D / 2.5D only")

    @property
    def cubic_dim(self) -> int:
        return _icbrt_exact(self.tensor_parallel_size, "3D")
