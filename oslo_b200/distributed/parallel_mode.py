"""Names of every process group the runtime can hold.

Parity: reference ``oslo/torch/distributed/parallel_mode.py:4-49`` (22 members;
member names and string values are part of the public surface and therefore kept).
"""
from enum import Enum


class ParallelMode(Enum):
    GLOBAL = "global"
    DATA = "data"
    MODEL = "model"
    PIPELINE = "pipe"
    TENSOR = "tensor"
    SEQUENCE = "sequence"
    SEQUENCE_DP = "sequence_dp"
    TENSOR_1D = "tensor_1d"
    TENSOR_2D = "tensor_2d"
    TENSOR_2D_ROW = "tensor_2d_row"
    TENSOR_2D_COL = "tensor_2d_col"
    TENSOR_2P5D = "tensor_2p5d"
    TENSOR_2P5D_ROW = "2p5d_row"
    TENSOR_2P5D_COL = "2p5d_col"
    TENSOR_2P5D_DEP = "2p5d_dep"
    TENSOR_2P5D_XZ = "2p5d_xz"
    TENSOR_3D = "tensor_3d"
    TENSOR_3D_INPUT = "tensor_3d_input"
    TENSOR_3D_WEIGHT = "tensor_3d_weight"
    TENSOR_3D_OUTPUT = "tensor_3d_output"
    EXPERT = "expert"

    def __repr__(self):  # compact in logs
        return f"ParallelMode.{self.name}"


#: The N-D "whole tensor group" modes; getters alias them to TENSOR
#: (reference ``parallel_context.py:1070-1088``).
ND_TENSOR_MODES = (
    ParallelMode.TENSOR_1D,
    ParallelMode.TENSOR_2D,
    ParallelMode.TENSOR_2P5D,
    ParallelMode.TENSOR_3D,
)
