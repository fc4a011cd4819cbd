from .expert_parallel import ExpertParallel
from .layers import ExpertParallelBehindBlock, ExpertParallelFrontBlock, Experts, TopKGate
from .mapping import Behind, ExpertParallelMapping, Front

__all__ = ["ExpertParallel", "TopKGate", "Experts", "ExpertParallelFrontBlock", "ExpertParallelBehindBlock",
           "ExpertParallelMapping", "Front", "Behind"]
