r"""
CUDA-graph capture of a whole training step.

The fused MoE path never reads a count on the host, so forward, backward, gradient
reduction and the optimizer update of a model built on it form a fixed launch sequence that
can be captured once and replayed; the reference cannot do this (its layer blocks the host
several times per call, ``fmoe/functions.py:46,68,71-73``).  Replay removes the Python and
launch overhead, which for a single MoE layer is as large as the GPU time itself.

    step = GraphedStep(lambda x: train_step(model, opt, x), example_input)
    loss = step(x)          # copies x into the static input, replays, returns the static loss

Rules for the captured function: no ``.item()`` / ``.cpu()`` / printing of device values, the
optimizer must be capturable (``torch.optim.Adam(..., capturable=True)``), and shapes must not
change between calls.  Run the model's first backward pass inside this helper (or on a side
stream): autograd binds every parameter's gradient-accumulation node to the stream of its first
use, and a node bound to the default stream cannot join a capture.  Gates that need host decisions (``SwipeGate``, ``FasterGate``) cannot be
captured.
"""
import torch


class GraphedStep:
    r"""Capture ``fn(static_input)`` into a CUDA graph after ``warmup`` eager runs on a side stream."""

    def __init__(self, fn, example_input, warmup=3, pool=None):
        self.fn = fn
        self.static_input = example_input.detach().clone()
        # Parameters were created on another stream than the capture stream: harmless here.
        try:
            torch.autograd.graph.set_warn_on_accumulate_grad_stream_mismatch(False)
        except AttributeError:
            pass
        self.graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self.static_output = fn(self.static_input)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        with torch.cuda.graph(self.graph, pool=pool):
            self.static_output = fn(self.static_input)

    def __call__(self, x=None, non_blocking=True):
        if x is not None and x.data_ptr() != self.static_input.data_ptr():
            self.static_input.copy_(x, non_blocking=non_blocking)
        self.graph.replay()
        return self.static_output
