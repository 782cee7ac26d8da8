r"""
Framework-agnostic checkpointing for expert-parallel models.

The reference only has Megatron checkpoints (``fmoe/megatron/checkpoint.py``); its
Transformer-XL example pickles the whole module (``examples/transformer-xl/train.py:516-523``).
Here any ``nn.Module`` whose parameters carry ``dp_comm`` tags can be saved and resumed:

    <dir>/step_{step:08d}/shared.pt              replicated tensors (``dp_comm != 'none'``), optimizer
                                                 state of those, RNG states, user metadata — written by
                                                 the first rank of the expert-parallel group
    <dir>/step_{step:08d}/experts_rank{r:04d}.pt every rank: its expert tensors (``dp_comm == 'none'``)
                                                 and their optimizer state
    <dir>/latest                                  the last completed step

Tensor names and shapes are those of ``state_dict()`` (expert layout
``experts.htoh4.weight [E, d_hidden, d_model]`` …), so a shard can be inspected or merged with
plain ``torch.load``.
"""
import os
import random

import numpy as np
import torch
import torch.distributed as dist

EXPERT_TAG = "none"


def _rank_world(group):
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def _barrier(group):
    if dist.is_available() and dist.is_initialized():
        dist.barrier(group)


def split_state_dict(module):
    r"""``(shared, experts)``: the module's ``state_dict`` split by the ``dp_comm`` tag."""
    tags = {name: getattr(p, "dp_comm", "dp") for name, p in module.named_parameters()}
    shared, experts = {}, {}
    for name, tensor in module.state_dict().items():
        (experts if tags.get(name) == EXPERT_TAG else shared)[name] = tensor.detach().cpu()
    return shared, experts


def _split_optimizer_state(module, optimizer):
    r"""Optimizer state split the same way; keys are parameter names instead of positions."""
    if optimizer is None:
        return None, None
    names = {id(p): n for n, p in module.named_parameters()}
    shared, experts = {}, {}
    for group in optimizer.param_groups:
        for p in group["params"]:
            name = names.get(id(p))
            st = optimizer.state.get(p)
            if name is None or not st:
                continue
            packed = {k: (v.detach().cpu() if torch.is_tensor(v) else v) for k, v in st.items()}
            (experts if getattr(p, "dp_comm", "dp") == EXPERT_TAG else shared)[name] = packed
    groups = [{k: v for k, v in g.items() if k != "params"} for g in optimizer.param_groups]
    return {"state": shared, "param_groups": groups}, {"state": experts}


def step_dir(directory, step):
    return os.path.join(directory, "step_{:08d}".format(step))


def save(directory, step, module, optimizer=None, group=None, extra=None):
    r"""Write one checkpoint; collective over ``group`` (the expert-parallel group)."""
    # A kernel that gave up on a peer (bounded wait) or dropped rows (bounded receive buffer)
    # only leaves a code in the device status word: never write a checkpoint of such a run.
    from .utils import check_device_status
    check_device_status()
    rank, _world = _rank_world(group)
    path = step_dir(directory, step)
    os.makedirs(path, exist_ok=True)
    shared, experts = split_state_dict(module)
    opt_shared, opt_experts = _split_optimizer_state(module, optimizer)
    torch.save({"model": experts, "optimizer": opt_experts, "step": step},
               os.path.join(path, "experts_rank{:04d}.pt".format(rank)))
    if rank == 0:
        rng = {"python": random.getstate(), "numpy": np.random.get_state(),
               "torch": torch.get_rng_state()}
        if torch.cuda.is_available():
            rng["cuda"] = torch.cuda.get_rng_state()
        torch.save({"model": shared, "optimizer": opt_shared, "rng": rng, "step": step,
                    "extra": extra}, os.path.join(path, "shared.pt"))
    _barrier(group)
    if rank == 0:
        with open(os.path.join(directory, "latest"), "w") as f:
            f.write(str(step))
    _barrier(group)
    return path


def latest_step(directory):
    try:
        with open(os.path.join(directory, "latest")) as f:
            return int(f.read().strip())
    except (OSError, ValueError):
        return None


def load(directory, module, optimizer=None, group=None, step=None, restore_rng=True):
    r"""Restore ``module`` (and ``optimizer``) in place; returns ``(step, extra)`` or ``(None, None)``."""
    if step is None:
        step = latest_step(directory)
    if step is None:
        return None, None
    rank, _world = _rank_world(group)
    path = step_dir(directory, step)
    shared = torch.load(os.path.join(path, "shared.pt"), map_location="cpu", weights_only=False)
    mine = torch.load(os.path.join(path, "experts_rank{:04d}.pt".format(rank)), map_location="cpu",
                      weights_only=False)
    state = dict(shared["model"])
    state.update(mine["model"])
    module.load_state_dict(state)
    if optimizer is not None and shared.get("optimizer") is not None:
        by_name = dict(module.named_parameters())
        merged = dict(shared["optimizer"]["state"])
        merged.update((mine.get("optimizer") or {}).get("state", {}))
        for name, packed in merged.items():
            p = by_name.get(name)
            if p is None:
                continue
            optimizer.state[p] = {k: (v.to(p.device) if torch.is_tensor(v) else v)
                                  for k, v in packed.items()}
        for group_now, saved in zip(optimizer.param_groups, shared["optimizer"]["param_groups"]):
            group_now.update(saved)
    if restore_rng and "rng" in shared:
        rng = shared["rng"]
        random.setstate(rng["python"])
        np.random.set_state(rng["numpy"])
        torch.set_rng_state(rng["torch"])
        if torch.cuda.is_available() and "cuda" in rng:
            torch.cuda.set_rng_state(rng["cuda"])
    _barrier(group)
    return shared.get("step", step), shared.get("extra")
