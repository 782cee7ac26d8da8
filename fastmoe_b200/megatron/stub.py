r"""
A stand-in for the parts of Megatron-LM that the adapter touches.

Megatron-LM is not a dependency of this package.  ``install(args, ...)`` registers modules
named ``megatron``, ``megatron.mpu``, ``megatron.checkpointing`` and ``megatron.utils`` with
exactly the objects the adapter imports — ``get_args``, ``get_num_microbatches``,
``print_rank_last``, ``is_last_rank``, process-group accessors, the tensor-parallel reduce,
checkpoint naming and a native-format ``save_checkpoint`` / ``load_checkpoint`` — so that
``fmoefy``, the patches, the DDP wrapper and the sharded checkpoints can be used (and tested)
from a plain PyTorch program such as ``examples/gpt/pretrain.py``.  With a real Megatron-LM on
the path nothing here is used.
"""
import os
import random
import sys
import types

import numpy as np
import torch
import torch.distributed as dist

_state = {}


def _world():
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def _rank():
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def install(args, data_parallel_group=None, tensor_parallel_group=None, pipeline_rank=0,
            pipeline_size=1, num_microbatches=1):
    r"""Create (or refresh) the stand-in modules around the namespace ``args``.

    Missing attributes of ``args`` get Megatron's defaults.  Groups default to: data parallel =
    world, tensor parallel = this rank alone.
    """
    defaults = dict(balance_strategy=None, balance_loss_weight=1.0, top_k=2, fmoe_num_experts=None,
                    distributed_experts=True, hidden_hidden_size=None, init_method_std=0.02,
                    tensor_model_parallel_size=1, pipeline_model_parallel_size=pipeline_size,
                    fp16=False, no_save_optim=False, no_load_optim=False, no_load_rng=False,
                    no_save_rng=False, finetune=False, save=None, load=None,
                    consumed_train_samples=0, consumed_valid_samples=0)
    for key, value in defaults.items():
        if not hasattr(args, key):
            setattr(args, key, value)
    args.rank = _rank()
    args.world_size = _world()
    if not hasattr(args, "data_parallel_size"):
        args.data_parallel_size = args.world_size // (args.tensor_model_parallel_size * pipeline_size)

    if dist.is_available() and dist.is_initialized():
        if data_parallel_group is None:
            data_parallel_group = dist.group.WORLD
        if tensor_parallel_group is None:
            tensor_parallel_group = None
            for r in range(_world()):
                g = dist.new_group([r])
                if r == _rank():
                    tensor_parallel_group = g
    _state.update(args=args, dp_group=data_parallel_group, tp_group=tensor_parallel_group,
                  pp_rank=pipeline_rank, pp_size=pipeline_size, num_microbatches=num_microbatches)

    megatron = types.ModuleType("megatron")
    mpu = types.ModuleType("megatron.mpu")
    ckpt = types.ModuleType("megatron.checkpointing")
    utils = types.ModuleType("megatron.utils")

    megatron.get_args = lambda: _state["args"]
    megatron.get_num_microbatches = lambda: _state["num_microbatches"]
    megatron.is_last_rank = lambda: _rank() == _world() - 1
    megatron.print_rank_last = lambda *a, **k: print(*a, **k, flush=True) if _rank() == _world() - 1 else None

    mpu.get_data_parallel_group = lambda: _state["dp_group"]
    mpu.get_tensor_model_parallel_group = lambda: _state["tp_group"]
    mpu.get_data_parallel_rank = lambda: dist.get_rank(_state["dp_group"]) if _state["dp_group"] is not None else 0
    mpu.get_data_parallel_world_size = lambda: dist.get_world_size(_state["dp_group"]) if _state["dp_group"] is not None else 1
    mpu.get_tensor_model_parallel_rank = lambda: dist.get_rank(_state["tp_group"]) if _state["tp_group"] is not None else 0
    mpu.get_tensor_model_parallel_world_size = lambda: dist.get_world_size(_state["tp_group"]) if _state["tp_group"] is not None else 1
    mpu.get_pipeline_model_parallel_rank = lambda: _state["pp_rank"]
    mpu.get_pipeline_model_parallel_world_size = lambda: _state["pp_size"]
    mpu.is_pipeline_last_stage = lambda: _state["pp_rank"] == _state["pp_size"] - 1
    mpu.is_pipeline_first_stage = lambda: _state["pp_rank"] == 0

    def reduce_from_tensor_model_parallel_region(x):
        group = _state["tp_group"]
        if group is None or dist.get_world_size(group) == 1:
            return x
        x = x.clone()
        dist.all_reduce(x, group=group)
        return x

    mpu.reduce_from_tensor_model_parallel_region = reduce_from_tensor_model_parallel_region

    def unwrap_model(model):
        models = model if isinstance(model, list) else [model]
        out = []
        for m in models:
            while hasattr(m, "module"):
                m = m.module
            out.append(m)
        return out

    utils.unwrap_model = unwrap_model

    # ---- native-format checkpointing (what Megatron itself writes on data-parallel rank 0)
    def get_checkpoint_name(checkpoints_path, iteration, release=False):
        directory = "release" if release else "iter_{:07d}".format(iteration)
        tp = mpu.get_tensor_model_parallel_rank()
        if _state["pp_size"] == 1:
            shard = "mp_rank_{:02d}".format(tp)
        else:
            shard = "mp_rank_{:02d}_{:03d}".format(tp, _state["pp_rank"])
        return os.path.join(checkpoints_path, directory, shard, "model_optim_rng.pt")

    def get_checkpoint_tracker_filename(checkpoints_path):
        return os.path.join(checkpoints_path, "latest_checkpointed_iteration.txt")

    def ensure_directory_exists(filename):
        os.makedirs(os.path.dirname(filename), exist_ok=True)

    def save_checkpoint(iteration, model, optimizer, lr_scheduler):
        a = _state["args"]
        model0 = unwrap_model(model)[0]
        state = {"args": a, "checkpoint_version": 3.0, "iteration": iteration,
                 "model": model0.state_dict_for_save_checkpoint()
                 if hasattr(model0, "state_dict_for_save_checkpoint") else model0.state_dict()}
        if not a.no_save_optim:
            if optimizer is not None:
                state["optimizer"] = optimizer.state_dict()
            if lr_scheduler is not None:
                state["lr_scheduler"] = lr_scheduler.state_dict()
        if not a.no_save_rng:
            state["random_rng_state"] = random.getstate()
            state["np_rng_state"] = np.random.get_state()
            state["torch_rng_state"] = torch.get_rng_state()
            if torch.cuda.is_available():
                state["cuda_rng_state"] = torch.cuda.get_rng_state()
        name = get_checkpoint_name(a.save, iteration)
        ensure_directory_exists(name)
        torch.save(state, name)
        if dist.is_available() and dist.is_initialized():
            dist.barrier()
        if _rank() == 0:
            with open(get_checkpoint_tracker_filename(a.save), "w") as f:
                f.write(str(iteration))
        if dist.is_available() and dist.is_initialized():
            dist.barrier()

    def load_checkpoint(model, optimizer, lr_scheduler, load_arg="load"):
        a = _state["args"]
        load_dir = getattr(a, load_arg)
        tracker = get_checkpoint_tracker_filename(load_dir)
        if not os.path.isfile(tracker):
            return 0
        with open(tracker) as f:
            iteration = int(f.read().strip())
        state = torch.load(get_checkpoint_name(load_dir, iteration), map_location="cpu", weights_only=False)
        unwrap_model(model)[0].load_state_dict(state["model"])
        if not a.finetune and not a.no_load_optim:
            if optimizer is not None and "optimizer" in state:
                optimizer.load_state_dict(state["optimizer"])
            if lr_scheduler is not None and "lr_scheduler" in state:
                lr_scheduler.load_state_dict(state["lr_scheduler"])
        if not a.finetune and not a.no_load_rng and "random_rng_state" in state:
            random.setstate(state["random_rng_state"])
            np.random.set_state(state["np_rng_state"])
            torch.set_rng_state(state["torch_rng_state"])
            if torch.cuda.is_available() and "cuda_rng_state" in state:
                torch.cuda.set_rng_state(state["cuda_rng_state"])
        if dist.is_available() and dist.is_initialized():
            dist.barrier()
        return state.get("iteration", iteration)

    ckpt.get_checkpoint_name = get_checkpoint_name
    ckpt.get_checkpoint_tracker_filename = get_checkpoint_tracker_filename
    ckpt.ensure_directory_exists = ensure_directory_exists
    ckpt.save_checkpoint = save_checkpoint
    ckpt.load_checkpoint = load_checkpoint
    ckpt.set_checkpoint_version = lambda v: None
    ckpt.check_checkpoint_args = lambda a: None
    ckpt.update_num_microbatches = lambda consumed_samples=0: None

    megatron.mpu = mpu
    megatron.checkpointing = ckpt
    megatron.utils = utils
    sys.modules["megatron"] = megatron
    sys.modules["megatron.mpu"] = mpu
    sys.modules["megatron.checkpointing"] = ckpt
    sys.modules["megatron.utils"] = utils
    return megatron


def uninstall():
    for name in ("megatron", "megatron.mpu", "megatron.checkpointing", "megatron.utils"):
        sys.modules.pop(name, None)
    _state.clear()
    # process groups derived from the stand-in's arguments are rebuilt on the next install
    from . import distributed as _distributed
    _distributed._registry.reset()  # pylint: disable=protected-access
