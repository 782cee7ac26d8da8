r"""Experiment directory and logging helpers of the Transformer-XL example, and a DataParallel
that gives the first GPU a smaller share of the batch.

Counterparts of ``examples/transformer-xl/utils/exp_utils.py`` and ``utils/data_parallel.py`` of
the reference: device 0 also holds the gathered outputs and the optimizer state, so with
``--multi_gpu --gpu0_bsz N`` it receives only ``N`` of the batch's sequences.
"""
import functools
import os
import shutil
import time

import torch
import torch.nn as nn
from torch.nn.parallel._functions import Scatter


def create_exp_dir(path, scripts_to_save=None):
    r"""Create ``path`` and keep copies of the given scripts under ``path/scripts``."""
    os.makedirs(path, exist_ok=True)
    if scripts_to_save:
        os.makedirs(os.path.join(path, "scripts"), exist_ok=True)
        for script in scripts_to_save:
            shutil.copyfile(script, os.path.join(path, "scripts", os.path.basename(script)))
    return get_logger(os.path.join(path, "log.txt"))


def _log(line, path=None, print_=True):
    if print_:
        print(line, flush=True)
    if path is not None:
        with open(path, "a", encoding="utf-8") as f:
            f.write(line + "\n")


def get_logger(path=None):
    r"""``log(line, print_=True)`` that also appends to ``path``."""
    return functools.partial(_log, path=path)


class Timer:
    def __init__(self):
        self.t0 = time.time()

    def elapsed(self):
        return time.time() - self.t0


def balanced_chunk_sizes(batch, n_devices, gpu0_bsz):
    r"""Sequences per device: ``gpu0_bsz`` for the first, the rest split as evenly as possible
    (earlier devices get the larger shares); devices that would get nothing are dropped."""
    assert 0 <= gpu0_bsz <= batch
    if n_devices == 1:
        return [batch]
    rest = batch - gpu0_bsz
    others = n_devices - 1
    base, extra = divmod(rest, others)
    sizes = [gpu0_bsz] + [base + (1 if i < extra else 0) for i in range(others)]
    return [s for s in sizes if s > 0] if gpu0_bsz > 0 else [0] + [s for s in sizes[1:] if s > 0]


class BalancedDataParallel(nn.DataParallel):
    r"""``nn.DataParallel`` whose first device takes ``gpu0_bsz`` entries of the batch dimension."""

    def __init__(self, gpu0_bsz, module, dim=0, device_ids=None):
        super().__init__(module, device_ids=device_ids, dim=dim)
        self.gpu0_bsz = gpu0_bsz

    def forward(self, *inputs, **kwargs):
        if not self.device_ids or len(self.device_ids) == 1:
            return super().forward(*inputs, **kwargs)
        batch = next(t for t in inputs if torch.is_tensor(t)).size(self.dim)
        sizes = balanced_chunk_sizes(batch, len(self.device_ids), min(self.gpu0_bsz, batch))
        device_ids = list(self.device_ids)
        if sizes[0] == 0:                 # device 0 only gathers
            sizes, device_ids = sizes[1:], device_ids[1:]
        device_ids = device_ids[:len(sizes)]

        def split(obj):
            if torch.is_tensor(obj):
                return Scatter.apply(device_ids, sizes, self.dim, obj)
            if isinstance(obj, (list, tuple)):
                return list(zip(*map(split, obj))) if obj else [() for _ in device_ids]
            return [obj for _ in device_ids]

        scattered = split(list(inputs))
        scattered = [tuple(s) for s in scattered]
        replicas = self.replicate(self.module, device_ids)
        outputs = self.parallel_apply(replicas, scattered, [kwargs] * len(scattered))
        return self.gather(outputs, self.output_device)
