"""Replay a fixed sequence of packed-linear calls as one CUDA graph.

A decoded token issues hundreds of small launches (the reference counts 497 matmuls per token,
src/ternel_mlx/layout.py:170-198); launching each from Python costs more than the kernels take.
``GraphedStep`` captures a callable once, with static input and output tensors, and replays it:
the caller copies new inputs in, replays, and reads the outputs.
"""

from __future__ import annotations

from typing import Callable, Sequence

import torch


class GraphedStep:
    """Capture ``fn(*static_inputs) -> tensor or tuple of tensors`` and replay it.

    ``fn`` must only launch work on the current stream (the packed ops do) and must not
    synchronise. The static inputs are owned by this object: ``__call__`` copies the given
    tensors (host or device) into them, replays the graph and returns the static outputs.
    """

    def __init__(self, fn: Callable, example_inputs: Sequence[torch.Tensor], warmup: int = 2) -> None:
        self.static_inputs = [t.clone() for t in example_inputs]
        side = torch.cuda.Stream(device=self.static_inputs[0].device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):               # warm up outside capture: workspaces, attributes
            for _ in range(warmup):
                fn(*self.static_inputs)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            out = fn(*self.static_inputs)
        self.static_outputs = out

    def __call__(self, *inputs: torch.Tensor):
        for dst, src in zip(self.static_inputs, inputs):
            dst.copy_(src, non_blocking=True)
        self.graph.replay()
        return self.static_outputs
