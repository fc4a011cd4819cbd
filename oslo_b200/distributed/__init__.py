from .parallel_context import ParallelContext
from .parallel_mode import ParallelMode
from .topology import Topology

__all__ = ["ParallelContext", "ParallelMode", "Topology"]
