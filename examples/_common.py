r"""Shared plumbing of the example entry points: process group, device, synthetic data."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def init_distributed():
    r"""One process per GPU (``torchrun``); falls back to a single process, CPU when no GPU exists."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if cuda:
            dist.init_process_group("nccl", device_id=device)
        else:
            dist.init_process_group("gloo")
    return rank, world, device


def max_over_ranks(value, device):
    if dist.is_available() and dist.is_initialized():
        t = torch.tensor([value], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)
    return float(value)


class Stopwatch:
    r"""CUDA-event (or wall-clock on CPU) timing of a block of steps."""

    def __init__(self, device):
        self.cuda = device.type == "cuda"

    def __enter__(self):
        import time
        if self.cuda:
            torch.cuda.synchronize()
            self.s = torch.cuda.Event(enable_timing=True)
            self.e = torch.cuda.Event(enable_timing=True)
            self.s.record()
        else:
            self.t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        import time
        if self.cuda:
            self.e.record()
            torch.cuda.synchronize()
            self.ms = self.s.elapsed_time(self.e)
        else:
            self.ms = (time.perf_counter() - self.t0) * 1e3
