"""oslo_b200: a Blackwell-native (sm_100a) large-model training framework with the capabilities and public
surface of EleutherAI/oslo (``ParallelContext``, ``ParallelMode``, ``ready`` and the parallel wrappers)."""
from oslo_b200.__version__ import __version__  # noqa: F401
from oslo_b200.distributed import ParallelContext, ParallelMode  # noqa: F401
from oslo_b200.utils.extensions import ready  # noqa: F401

__all__ = ["ParallelContext", "ParallelMode", "ready"]
