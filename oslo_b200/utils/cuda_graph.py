"""Whole-step CUDA-graph capture: one graph launch replaces the thousands of kernel launches of a training step.

At tensor-parallel sizes of 4-8 a 1.3B-parameter step leaves each GPU ~40 ms of kernels but costs the host ~80 ms of
launch work, so the step is host-bound; replaying a captured graph removes that.  ``GraphedStep(fn, example_inputs)``
warms ``fn`` up eagerly, captures one call, and afterwards ``graphed(*inputs)`` copies the inputs into the static
buffers, replays and returns the static outputs.

What makes this repository's step capturable:
* kernels take raw pointers; tensor maps are encoded on the host from addresses that are stable inside a graph pool;
* optimizer tensor tables are uploaded from pinned memory with an async copy (legal during capture);
* ``FusedAdam(capturable=True)`` keeps the step count on the device;
* the fused-collective epochs live in device memory and are advanced by stream-ordered increments, and
  ``pad_to_even`` keeps the double-buffer parity identical from replay to replay.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch


class GraphedStep:
    def __init__(self, fn: Callable, example_inputs: Sequence[torch.Tensor], warmup: int = 3, before_capture_end: Callable = None):
        self.fn = fn
        self.static_inputs = [t.clone() for t in example_inputs]
        self.graph = None
        self.static_outputs = None
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                out = fn(*self.static_inputs)
                if before_capture_end is not None:
                    before_capture_end()
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            out = fn(*self.static_inputs)
            if before_capture_end is not None:
                before_capture_end()
        self.graph = graph
        self.static_outputs = out

    def __call__(self, *inputs):
        for dst, src in zip(self.static_inputs, inputs):
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src, non_blocking=True)
        self.graph.replay()
        return self.static_outputs


def try_graphed_step(fn, example_inputs, warmup: int = 3, before_capture_end=None, on_failure=None):
    """``GraphedStep`` if capture works, else ``fn`` itself (the reason is passed to ``on_failure``)."""
    try:
        return GraphedStep(fn, example_inputs, warmup, before_capture_end)
    except Exception as e:  # capture is an optimisation; the eager step is always valid
        torch.cuda.synchronize()
        if on_failure is not None:
            on_failure(e)
        return None
