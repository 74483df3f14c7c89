"""CUDA-graph replay of a fixed step.

A decoder layer at a tensor-parallel degree of 4 or 8 is a few dozen kernels of 10-50 microseconds
each: launched one by one from Python the step is bound by the host, not by the GPU.  Everything in
this package runs on the caller's stream without host synchronisation (per-tensor scales, run sizes of
the MoE dispatch and GEMM alphas stay on the device), so a whole step - NCCL collectives included - can
be captured once and replayed as one graph launch.
"""
from __future__ import annotations

import torch


class GraphedStep:
    """Captures `fn()` (no arguments: it reads static input tensors the caller refills in place) after a
    few eager warm-up calls on a side stream, and replays it.  `fn`'s return value is kept; every replay
    overwrites it in place."""

    def __init__(self, fn, warmup: int = 3, device=None):
        self.fn = fn
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        side = torch.cuda.Stream(dev)
        cur = torch.cuda.current_stream(dev)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):      # allocations, kernel attributes, communicators: all set up here
                fn()
        cur.wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.out = fn()

    def __call__(self):
        self.graph.replay()
        return self.out
