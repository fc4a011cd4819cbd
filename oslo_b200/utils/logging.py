"""Rank-aware logger (parity: oslo/torch/utils/logging/logger.py:8-110).

``get_dist_logger(name)`` returns one logger per name; ``logger.info(msg, ranks=[0])`` prints on the listed global
ranks only; ``attach_file_handler(path, suffix)`` adds ``rank_{r}[_suffix].log``.
"""
from __future__ import annotations

import logging
import os
from typing import Dict, List, Optional

import torch.distributed as dist

_LOGGERS: Dict[str, "DistributedLogger"] = {}


class DistributedLogger:
    def __init__(self, name: str):
        self._name = name
        self._logger = logging.getLogger(name)
        if not self._logger.handlers:
            h = logging.StreamHandler()
            h.setFormatter(logging.Formatter("[%(asctime)s] %(levelname)s %(name)s: %(message)s"))
            self._logger.addHandler(h)
        self._logger.setLevel(logging.INFO)
        self._logger.propagate = False

    @staticmethod
    def get_instance(name: str) -> "DistributedLogger":
        if name not in _LOGGERS:
            _LOGGERS[name] = DistributedLogger(name)
        return _LOGGERS[name]

    @staticmethod
    def _rank() -> int:
        return dist.get_rank() if dist.is_available() and dist.is_initialized() else int(os.environ.get("RANK", 0))

    def set_level(self, level: str):
        self._logger.setLevel(getattr(logging, level.upper()))

    def attach_file_handler(self, path: str, mode: str = "a", level: str = "INFO", suffix: Optional[str] = None):
        os.makedirs(path, exist_ok=True)
        name = f"rank_{self._rank()}" + (f"_{suffix}" if suffix else "") + ".log"
        h = logging.FileHandler(os.path.join(path, name), mode)
        h.setLevel(getattr(logging, level.upper()))
        h.setFormatter(logging.Formatter("[%(asctime)s] %(levelname)s %(name)s: %(message)s"))
        self._logger.addHandler(h)

    def _log(self, level: str, message: str, ranks: Optional[List[int]] = None):
        if ranks is None or self._rank() in ranks:
            getattr(self._logger, level)(message)

    def info(self, message, ranks=None):
        self._log("info", message, ranks)

    def warning(self, message, ranks=None):
        self._log("warning", message, ranks)

    def debug(self, message, ranks=None):
        self._log("debug", message, ranks)

    def error(self, message, ranks=None):
        self._log("error", message, ranks)


def get_dist_logger(name: str = "oslo_b200") -> DistributedLogger:
    return DistributedLogger.get_instance(name)


def log_dist(message: str, rank: int = 0, level: str = "info"):
    get_dist_logger()._log(level, message, None if rank < 0 else [rank])
