"""Per-ParallelMode random-number-generator states.

Each mode owns one RNG state; ``seed(mode)`` temporarily switches the active
generator so that, e.g., dropout inside a tensor-parallel region draws different
numbers on every TP rank while data-parallel replicas stay identical.

Works on CPU (``torch.get_rng_state``) and CUDA (``torch.cuda.get_rng_state``),
unlike the reference which is CUDA-only (``_seed/seed_manager.py:31-55``).
Parity: ``oslo/torch/distributed/_seed/helper.py:13-94``.
"""
from __future__ import annotations

import functools
from contextlib import contextmanager
from typing import Dict, Optional

import torch

from .parallel_mode import ParallelMode


def _use_cuda() -> bool:
    return torch.cuda.is_available() and torch.cuda.is_initialized()


def _get_state() -> torch.Tensor:
    return torch.cuda.get_rng_state() if _use_cuda() else torch.get_rng_state()


def _set_state(state: torch.Tensor) -> None:
    if _use_cuda():
        torch.cuda.set_rng_state(state)
    else:
        torch.set_rng_state(state)


def _manual_seed(seed: int) -> None:
    if _use_cuda():
        torch.cuda.manual_seed(seed)
    else:
        torch.manual_seed(seed)


class SeedManager:
    def __init__(self):
        self._current_mode: Optional[ParallelMode] = None
        self._seeds: Dict[ParallelMode, int] = {}
        self._states: Dict[ParallelMode, torch.Tensor] = {}

    @property
    def current_mode(self):
        return self._current_mode

    @property
    def seeds(self):
        return self._seeds

    @property
    def seed_states(self):
        return self._states

    def set_state(self, mode: ParallelMode, state: torch.Tensor):
        if mode not in self._states:
            raise KeyError(f"{mode} has no registered seed")
        self._states[mode] = state

    def set_mode(self, mode: ParallelMode):
        if mode not in self._states:
            raise KeyError(f"{mode} has no registered seed")
        if self._current_mode is not None:
            self._states[self._current_mode] = _get_state()
        self._current_mode = mode
        _set_state(self._states[mode])

    def add_seed(self, mode: ParallelMode, seed: int, overwrite: bool = False):
        if not isinstance(mode, ParallelMode):
            raise TypeError("mode must be a ParallelMode")
        if mode in self._states and not overwrite:
            raise ValueError(f"seed for {mode} already registered")
        saved = _get_state()
        _manual_seed(seed)
        self._states[mode] = _get_state()
        self._seeds[mode] = seed
        _set_state(saved)

    def reset(self):
        self._current_mode = None
        self._seeds = {}
        self._states = {}


_MANAGER = SeedManager()


def get_seeds():
    return _MANAGER.seeds


def get_states(copy: bool = False):
    states = _MANAGER.seed_states
    if copy:
        return {m: s.clone() for m, s in states.items()}
    return states


def get_current_mode():
    return _MANAGER.current_mode


def add_seed(parallel_mode: ParallelMode, seed: int, overwrite: bool = False):
    _MANAGER.add_seed(parallel_mode, seed, overwrite)


def set_mode(parallel_mode: ParallelMode):
    _MANAGER.set_mode(parallel_mode)


def set_seed_states(parallel_mode: ParallelMode, state: torch.Tensor):
    _MANAGER.set_state(parallel_mode, state)


def sync_states():
    """Store the live generator state back into the current mode's slot."""
    mode = get_current_mode()
    if mode is not None:
        set_seed_states(mode, _get_state())


@contextmanager
def seed(parallel_mode: ParallelMode):
    previous = _MANAGER.current_mode
    try:
        _MANAGER.set_mode(parallel_mode)
        yield
    finally:
        if previous is not None:
            _MANAGER.set_mode(previous)


def with_seed(func, parallel_mode: ParallelMode):
    @functools.wraps(func)
    def wrapper(*args, **kwargs):
        with seed(parallel_mode):
            return func(*args, **kwargs)

    return wrapper


def moe_set_seed(parallel_context, seed_value: int):
    """Expert weights must differ per rank: seed with ``seed + global_rank``."""
    rank = parallel_context.get_global_rank()
    _manual_seed(seed_value + rank)
    return seed_value + rank


def reset_seeds():
    _MANAGER.reset()
