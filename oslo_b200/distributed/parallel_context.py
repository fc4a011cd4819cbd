"""Process-group runtime: one object that owns every communicator of a job.

``ParallelContext.from_torch(...)`` reads the torchrun environment, initialises
``torch.distributed`` (NCCL on GPUs, gloo on CPU), computes the rank topology
with :mod:`oslo_b200.distributed.topology` and creates one process group per
*distinct* rank list (several modes that share ranks share a communicator, so an
8-GPU job creates a dozen NCCL communicators instead of ~2 x modes x groups).
When the main backend is NCCL, a gloo twin of each group is created lazily-free
at start-up for host-side control traffic (``get_cpu_group``).

Nothing in this file requires a GPU: with ``backend="gloo"`` the whole runtime
runs on CPU, which the reference cannot do (it calls ``.cuda()`` unconditionally,
``oslo/torch/distributed/parallel_context.py:943-950``).

Parity: public constructor/getter surface of
``oslo/torch/distributed/parallel_context.py:182-1088``.
"""
from __future__ import annotations

import datetime
import os
import random
import weakref
from typing import Dict, List, Optional, Tuple, Union

import numpy as np
import torch
import torch.distributed as dist

from . import seed as _seed
from .parallel_mode import ND_TENSOR_MODES, ParallelMode
from .topology import Topology

_MODE_ALIASES = {
    "1d": ParallelMode.TENSOR_1D,
    "2d": ParallelMode.TENSOR_2D,
    "2.5d": ParallelMode.TENSOR_2P5D,
    "2p5d": ParallelMode.TENSOR_2P5D,
    "3d": ParallelMode.TENSOR_3D,
}


def _as_mode(mode) -> Optional[ParallelMode]:
    if mode is None or isinstance(mode, ParallelMode):
        return mode
    if isinstance(mode, str):
        key = mode.lower()
        if key in _MODE_ALIASES:
            return _MODE_ALIASES[key]
        for m in ParallelMode:
            if m.value == key or m.name.lower() == key:
                return m
    raise ValueError(f"unknown tensor_parallel_mode {mode!r}")


class ParallelContext:
    """Holds ranks, world sizes and communicators for every :class:`ParallelMode`."""

    _instances: List["weakref.ReferenceType[ParallelContext]"] = []

    # ------------------------------------------------------------ constructors
    @classmethod
    def get_context(cls, idx: int = -1) -> Optional["ParallelContext"]:
        if not cls._instances:
            return None
        if idx < 0:
            idx += len(cls._instances)
        if not 0 <= idx < len(cls._instances):
            raise IndexError("parallel context index out of range")
        return cls._instances[idx]()

    @classmethod
    def from_torch(
        cls,
        data_parallel_size: int = 1,
        sequence_parallel_size: int = 1,
        expert_parallel_size: int = 1,
        pipeline_parallel_size: int = 1,
        tensor_parallel_size: int = 1,
        tensor_parallel_depth: Optional[int] = None,
        tensor_parallel_mode: Optional[Union[ParallelMode, str]] = ParallelMode.TENSOR_1D,
        backend: str = "nccl",
        seed: int = 42,
        **kwargs,
    ) -> "ParallelContext":
        """Build from the environment written by ``torchrun`` / ``torch.distributed.run``.  A plain ``python script.py``
        (no ``RANK`` / ``WORLD_SIZE``) is a job of one process on a free local port."""
        env = os.environ
        if "RANK" not in env and "WORLD_SIZE" not in env:
            import socket

            with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as sock:
                sock.bind(("127.0.0.1", 0))
                free = sock.getsockname()[1]
            env = {"RANK": "0", "WORLD_SIZE": "1", "LOCAL_RANK": "0", "LOCAL_WORLD_SIZE": "1", "MASTER_ADDR": "127.0.0.1",
                   "MASTER_PORT": env.get("MASTER_PORT", str(free))}
        return cls(
            rank=int(env["RANK"]),
            local_rank=int(env.get("LOCAL_RANK", env["RANK"])),
            world_size=int(env["WORLD_SIZE"]),
            local_world_size=int(env.get("LOCAL_WORLD_SIZE", env["WORLD_SIZE"])),
            host=env.get("MASTER_ADDR", "127.0.0.1"),
            port=int(env.get("MASTER_PORT", "29500")),
            data_parallel_size=data_parallel_size,
            sequence_parallel_size=sequence_parallel_size,
            expert_parallel_size=expert_parallel_size,
            pipeline_parallel_size=pipeline_parallel_size,
            tensor_parallel_size=tensor_parallel_size,
            tensor_parallel_depth=tensor_parallel_depth,
            tensor_parallel_mode=tensor_parallel_mode,
            backend=backend,
            seed=seed,
            **kwargs,
        )

    @classmethod
    def from_slurm(cls, host: str, port: int, **kwargs) -> "ParallelContext":
        """Build from SLURM variables (``SLURM_PROCID``, ``SLURM_NPROCS``, ``SLURM_GPUS_ON_NODE``)."""
        env = os.environ
        rank = int(env["SLURM_PROCID"])
        world = int(env["SLURM_NPROCS"])
        per_node = int(env.get("SLURM_GPUS_ON_NODE", world))
        return cls(
            rank=rank,
            local_rank=rank % per_node if per_node else None,
            world_size=world,
            local_world_size=per_node,
            host=host,
            port=port,
            **cls._fill_defaults(kwargs),
        )

    @classmethod
    def from_openmpi(cls, host: str, port: int, **kwargs) -> "ParallelContext":
        """Build from Open MPI variables (``OMPI_COMM_WORLD_*``)."""
        env = os.environ
        return cls(
            rank=int(env["OMPI_COMM_WORLD_RANK"]),
            local_rank=int(env["OMPI_COMM_WORLD_LOCAL_RANK"]),
            world_size=int(env["OMPI_COMM_WORLD_SIZE"]),
            local_world_size=int(env["OMPI_COMM_WORLD_LOCAL_SIZE"]),
            host=host,
            port=port,
            **cls._fill_defaults(kwargs),
        )

    @staticmethod
    def _fill_defaults(kwargs):
        out = dict(
            data_parallel_size=1,
            sequence_parallel_size=1,
            expert_parallel_size=1,
            pipeline_parallel_size=1,
            tensor_parallel_size=1,
            tensor_parallel_depth=None,
            tensor_parallel_mode=ParallelMode.TENSOR_1D,
            backend="nccl",
            seed=42,
        )
        out.update(kwargs)
        return out

    def __init__(
        self,
        rank: int,
        local_rank: Optional[int],
        world_size: int,
        local_world_size: int,
        host: str,
        port: int,
        data_parallel_size: int = 1,
        sequence_parallel_size: int = 1,
        expert_parallel_size: Union[int, dict] = 1,
        pipeline_parallel_size: int = 1,
        tensor_parallel_size: int = 1,
        tensor_parallel_depth: Optional[int] = None,
        tensor_parallel_mode: Optional[Union[ParallelMode, str]] = ParallelMode.TENSOR_1D,
        backend: str = "nccl",
        seed: int = 42,
        expert_overlay: Optional[bool] = None,
        timeout_s: Optional[float] = None,
    ):
        tensor_parallel_mode = _as_mode(tensor_parallel_mode)
        self._pyramid_expert_sizes = expert_parallel_size if isinstance(expert_parallel_size, dict) else None
        ep_scalar = 1 if self._pyramid_expert_sizes is not None else int(expert_parallel_size)
        base = data_parallel_size * pipeline_parallel_size * tensor_parallel_size * sequence_parallel_size
        if expert_overlay is None:
            # EP that cannot multiply into the world size but divides DP overlays the DP ranks.
            expert_overlay = ep_scalar > 1 and world_size == base and data_parallel_size % ep_scalar == 0
        self.topology = Topology(
            world_size=world_size,
            data_parallel_size=data_parallel_size,
            pipeline_parallel_size=pipeline_parallel_size,
            tensor_parallel_size=tensor_parallel_size,
            sequence_parallel_size=sequence_parallel_size,
            expert_parallel_size=ep_scalar,
            tensor_parallel_mode=tensor_parallel_mode,
            tensor_parallel_depth=tensor_parallel_depth,
            expert_overlay=expert_overlay,
        ).validate()

        self.data_parallel_size = data_parallel_size
        self.sequence_parallel_size = sequence_parallel_size
        self.expert_parallel_size = expert_parallel_size
        self.pipeline_parallel_size = pipeline_parallel_size
        self.tensor_parallel_size = tensor_parallel_size
        self.tensor_parallel_mode = tensor_parallel_mode
        self.tensor_parallel_depth = tensor_parallel_depth
        self.local_world_size = local_world_size
        self.backend = backend
        self.host, self.port = host, port
        self.seed = seed

        self._global_rank = rank
        self._local_ranks: Dict[ParallelMode, int] = {}
        self._world_sizes: Dict[ParallelMode, int] = {}
        self._groups: Dict[ParallelMode, dist.ProcessGroup] = {}
        self._cpu_groups: Dict[ParallelMode, dist.ProcessGroup] = {}
        self._ranks_in_group: Dict[ParallelMode, List[int]] = {}
        self._expert_parallel_info: Dict[str, dict] = {}
        self._group_cache: Dict[Tuple[int, ...], Tuple[dist.ProcessGroup, dist.ProcessGroup]] = {}
        self._ranks_to_device: Dict[tuple, int] = {}
        self._owns_default_group = False

        self.use_cuda = backend == "nccl" and torch.cuda.is_available()
        if self.use_cuda:
            self.set_device(local_rank)
        self.device = torch.device("cuda", torch.cuda.current_device()) if self.use_cuda else torch.device("cpu")

        self.init_global_dist(rank, world_size, backend, host, port, timeout_s)
        self.init_parallel_groups()
        self.set_seed(seed)
        self.make_ranks_to_devices()

        ParallelContext._instances.append(weakref.ref(self))

    # ---------------------------------------------------------------- bring-up
    def init_global_dist(self, rank, world_size, backend, host, port, timeout_s=None):
        if not dist.is_initialized():
            kwargs = {}
            if timeout_s is not None:
                kwargs["timeout"] = datetime.timedelta(seconds=timeout_s)
            if self.use_cuda:
                kwargs["device_id"] = self.device
            dist.init_process_group(
                backend=backend,
                init_method=f"tcp://{host}:{port}",
                rank=rank,
                world_size=world_size,
                **kwargs,
            )
            self._owns_default_group = True
        elif dist.get_world_size() != world_size or dist.get_rank() != rank:
            raise RuntimeError("torch.distributed is already initialised with a different rank/world size")

    def _make_group(self, ranks: List[int]):
        """One communicator (and one gloo twin) per distinct rank list, shared by modes."""
        key = tuple(ranks)
        hit = self._group_cache.get(key)
        if hit is not None:
            return hit
        if len(ranks) == dist.get_world_size():
            group = dist.group.WORLD
        else:
            group = dist.new_group(ranks)
        if self.backend != "gloo":
            cpu_group = dist.new_group(ranks, backend="gloo")
        else:
            cpu_group = group
        self._group_cache[key] = (group, cpu_group)
        return group, cpu_group

    def _register(self, mode: ParallelMode, ranks: List[int], group, cpu_group):
        self._local_ranks[mode] = ranks.index(self._global_rank)
        self._world_sizes[mode] = len(ranks)
        self._groups[mode] = group
        self._cpu_groups[mode] = cpu_group
        self._ranks_in_group[mode] = list(ranks)

    def init_parallel_groups(self):
        topo = self.topology
        for mode in topo.active_modes():
            mine = None
            # new_group is collective over the whole world: every rank walks every group.
            for ranks in topo.groups(mode):
                group, cpu_group = self._make_group(ranks)
                if self._global_rank in ranks:
                    mine = (ranks, group, cpu_group)
            if mine is not None:
                self._register(mode, *mine)
        if self._pyramid_expert_sizes is not None:
            # per-layer ("pyramid") expert group sizes: {"enc": {layer_id: ep}, "dec": {...}}
            for stack, per_layer in self._pyramid_expert_sizes.items():
                self._expert_parallel_info[stack] = {}
                for layer_id, ep in per_layer.items():
                    for ranks in topo.expert_groups(ep):
                        group, cpu_group = self._make_group(ranks)
                        if self._global_rank in ranks:
                            self._expert_parallel_info[stack][layer_id] = dict(
                                local_rank=ranks.index(self._global_rank),
                                group_world_size=len(ranks),
                                process_group=group,
                                cpu_group=cpu_group,
                                ranks_in_group=list(ranks),
                            )

    def set_device(self, device_ordinal: Optional[int] = None):
        if not torch.cuda.is_available():
            return
        if device_ordinal is None:
            device_ordinal = self._global_rank % torch.cuda.device_count()
        torch.cuda.set_device(device_ordinal % torch.cuda.device_count())

    def set_seed(self, seed: int):
        """Seed python/numpy/torch; DATA seed equal on all ranks, TENSOR seed = seed + tp_rank + 1024*pp_rank."""
        random.seed(seed)
        np.random.seed(seed % (2**32))
        torch.manual_seed(seed)
        _seed.reset_seeds()
        _seed.add_seed(ParallelMode.DATA, seed)
        tp_rank = self._local_ranks.get(ParallelMode.TENSOR, 0)
        pp_rank = self._local_ranks.get(ParallelMode.PIPELINE, 0)
        _seed.add_seed(ParallelMode.TENSOR, seed + tp_rank + 1024 * pp_rank)
        _seed.set_mode(ParallelMode.DATA)

    def make_ranks_to_devices(self):
        """Map ``{mode: local rank}`` tuples to global ranks, computed from the topology (no collective)."""
        modes = list(self._local_ranks.keys())
        self._device_key_modes = modes
        topo = self.topology
        for r in range(topo.world_size):
            key = tuple((m, topo.group_of(m, r).index(r)) for m in modes)
            self._ranks_to_device[key] = r

    def ranks2device(self, ranks: Dict[ParallelMode, int]) -> Optional[int]:
        """Global rank whose local ranks equal ``ranks`` (missing modes default to this rank's)."""
        key = tuple(
            (m, ranks[m] if m in ranks else self._local_ranks[m]) for m in self._device_key_modes
        )
        return self._ranks_to_device.get(key)

    # ------------------------------------------------------------------ getters
    def _resolve(self, mode: ParallelMode) -> ParallelMode:
        if not isinstance(mode, ParallelMode):
            raise TypeError(f"expected ParallelMode, got {type(mode)}")
        if mode in ND_TENSOR_MODES:
            return ParallelMode.TENSOR
        return mode

    def is_initialized(self, parallel_mode: ParallelMode) -> bool:
        return self._resolve(parallel_mode) in self._groups

    def get_global_rank(self) -> int:
        return self._global_rank

    def get_world_size(self, parallel_mode: ParallelMode) -> int:
        return self._world_sizes[self._resolve(parallel_mode)]

    def get_local_rank(self, parallel_mode: ParallelMode) -> int:
        return self._local_ranks[self._resolve(parallel_mode)]

    def get_local_ranks(self) -> Dict[ParallelMode, int]:
        return self._local_ranks

    def get_group(self, parallel_mode: ParallelMode):
        return self._groups[self._resolve(parallel_mode)]

    def get_cpu_group(self, parallel_mode: ParallelMode):
        return self._cpu_groups[self._resolve(parallel_mode)]

    def get_ranks_in_group(self, parallel_mode: ParallelMode) -> List[int]:
        return self._ranks_in_group[self._resolve(parallel_mode)]

    def get_next_global_rank(self, parallel_mode: ParallelMode) -> int:
        ranks = self.get_ranks_in_group(parallel_mode)
        return ranks[(self.get_local_rank(parallel_mode) + 1) % len(ranks)]

    def get_prev_global_rank(self, parallel_mode: ParallelMode) -> int:
        ranks = self.get_ranks_in_group(parallel_mode)
        return ranks[(self.get_local_rank(parallel_mode) - 1) % len(ranks)]

    def is_first_rank(self, parallel_mode: ParallelMode) -> bool:
        return self.get_local_rank(parallel_mode) == 0

    def is_last_rank(self, parallel_mode: ParallelMode) -> bool:
        return self.get_local_rank(parallel_mode) == self.get_world_size(parallel_mode) - 1

    def get_expert_parallel_info(self, stack: str, layer_id) -> dict:
        return self._expert_parallel_info[stack][layer_id]

    def local_ranks_to_global_rank(self, *, dp_rank: int, pp_rank: int, tp_rank: int) -> int:
        topo = self.topology
        block = topo.world_size // topo.data_parallel_size
        return dp_rank * block + pp_rank * (block // topo.pipeline_parallel_size) + tp_rank

    def need_tensor_group_sync(self) -> bool:
        return self.tensor_parallel_size > 1

    # extra helpers of the new runtime -------------------------------------
    @property
    def summa_dim(self) -> int:
        return self.topology.summa_dim

    @property
    def cubic_dim(self) -> int:
        return self.topology.cubic_dim

    # manual registration hooks kept for API parity ---------------------------
    def add_world_size(self, parallel_mode, world_size):
        self._world_sizes[parallel_mode] = world_size

    def add_local_rank(self, parallel_mode, rank):
        self._local_ranks[parallel_mode] = rank

    def add_group(self, parallel_mode, group):
        self._groups[parallel_mode] = group

    def add_cpu_group(self, parallel_mode, group):
        self._cpu_groups[parallel_mode] = group

    def add_ranks_in_group(self, parallel_mode, ranks):
        self._ranks_in_group[parallel_mode] = ranks

    def destroy(self):
        """Tear down every communicator created by this context."""
        seen = set()
        for group, cpu_group in self._group_cache.values():
            for g in (group, cpu_group):
                if g is dist.group.WORLD or id(g) in seen:
                    continue
                seen.add(id(g))
                try:
                    dist.destroy_process_group(g)
                except Exception:
                    pass
        if self._owns_default_group and dist.is_initialized():
            dist.destroy_process_group()
        self._groups.clear()
        self._cpu_groups.clear()
        self._group_cache.clear()
