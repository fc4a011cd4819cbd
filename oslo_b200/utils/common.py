"""Small helpers (parity: oslo/torch/utils/common.py:5-19, version.py)."""
import random
import socket

import numpy as np
import torch


def get_free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def set_seed(seed: int):
    random.seed(seed)
    np.random.seed(seed % (2**32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def torch_version():
    major, minor = torch.__version__.split(".")[:2]
    return int(major), int(minor)
