r"""
Megatron checkpoints with expert-parallel shards (parity: ``fmoe/megatron/checkpoint.py``).

Layout on disk (identical to the reference):

    <save>/latest_checkpointed_iteration.txt
    <save>/iter_{it:07d}/mp_rank_{tp:02d}[_{pp:03d}]/model_optim_rng.pt               data-parallel rank 0: everything
    <save>/iter_{it:07d}/mp_rank_{tp:02d}[_{pp:03d}]_dp_rank_{dp:04d}/model_optim_rng.pt   other ranks: expert tensors
                                                                                   (``dp_comm == 'none'``) and their optimizer state

Data-parallel rank 0 goes through Megatron's own ``save_checkpoint`` / ``load_checkpoint``;
every other rank writes only what differs from rank 0 — its experts — and on load overlays its
shard on rank 0's file (``merge_state_dict``).  Interleaved pipeline stages are not supported.
"""
import os
import random
from collections import OrderedDict

import numpy as np
import torch

EXPERT_DP_COMM = "none"


def get_fmoe_checkpoint_name(checkpoints_path, iteration, release=False, data_parallel_rank=-1):
    r"""File of one data-parallel rank; rank 0 uses Megatron's native name."""
    from megatron import mpu
    from megatron.checkpointing import get_checkpoint_name
    if data_parallel_rank == -1:
        data_parallel_rank = mpu.get_data_parallel_rank()
    if data_parallel_rank == 0:
        return get_checkpoint_name(checkpoints_path, iteration, release)
    directory = "release" if release else "iter_{:07d}".format(iteration)
    tp = mpu.get_tensor_model_parallel_rank()
    if mpu.get_pipeline_model_parallel_world_size() == 1:
        shard = "mp_rank_{:02d}_dp_rank_{:04d}".format(tp, data_parallel_rank)
    else:
        shard = "mp_rank_{:02d}_{:03d}_dp_rank_{:04d}".format(
            tp, mpu.get_pipeline_model_parallel_rank(), data_parallel_rank)
    return os.path.join(checkpoints_path, directory, shard, "model_optim_rng.pt")


def _unwrap(model):
    try:
        from megatron import utils
        return utils.unwrap_model(model)
    except (ImportError, AttributeError):
        while hasattr(model, "module"):
            model = model.module
        return [model]


def extract_expert_param(state_dict, expert_dp_comm=EXPERT_DP_COMM):
    r"""Sub-dictionary (same nesting) of the tensors tagged ``dp_comm == expert_dp_comm``."""
    out = state_dict.__class__()
    for key, value in state_dict.items():
        if isinstance(value, (OrderedDict, dict)):
            sub = extract_expert_param(value, expert_dp_comm)
            if len(sub) > 0:
                out[key] = sub
        elif getattr(value, "dp_comm", None) == expert_dp_comm:
            out[key] = value.detach()
    return out


def _is_expert(param):
    return getattr(param, "dp_comm", None) == EXPERT_DP_COMM


def save_checkpoint(iteration, model, optimizer, lr_scheduler):
    r"""Save with expert parallelism: rank 0 natively, other data-parallel ranks their experts."""
    from megatron import get_args, mpu, print_rank_last
    if mpu.get_data_parallel_rank() == 0:
        from megatron.checkpointing import save_checkpoint as save_native
        save_native(iteration, model, optimizer, lr_scheduler)
        return

    args = get_args()
    model = _unwrap(model)
    assert len(model) == 1, "interleaved pipelining is not supported (len(model) must be 1)"
    print_rank_last("saving checkpoint at iteration {:7d} to {}".format(iteration, args.save))

    state = {"model": extract_expert_param(model[0].state_dict_for_save_checkpoint(keep_vars=True))}

    if not args.no_save_optim and optimizer is not None:
        opt_state = optimizer.state_dict()
        inner = opt_state["optimizer"] if args.fp16 else opt_state
        index = 0
        for group in optimizer.optimizer.param_groups:
            for param in group["params"]:
                if not _is_expert(param):
                    # replicated parameter: data-parallel rank 0 has saved its state
                    inner["state"].pop(index, None)
                index += 1
        inner.pop("param_groups", None)
        if args.fp16:
            # keep only the fp32 master copies of expert parameters (positions preserved)
            opt_state["fp32_from_fp16_params"] = [
                [p if _is_expert(p) else None for p in group]
                for group in opt_state["fp32_from_fp16_params"]]
        state["optimizer"] = opt_state

    name = get_fmoe_checkpoint_name(args.save, iteration)
    os.makedirs(os.path.dirname(name), exist_ok=True)
    torch.save(state, name)
    # Rank 0 of the world (a data-parallel rank 0) writes the tracker inside the native save;
    # the barriers there and here pair up.
    torch.distributed.barrier()
    torch.distributed.barrier()


def merge_state_dict(state_dict_rank0, state_dict_local, fp16):
    r"""Overlay the expert shard ``state_dict_local`` on rank 0's full state."""

    def merge_model(full, shard):
        for key, value in shard.items():
            if isinstance(value, (OrderedDict, dict)):
                merge_model(full[key], value)
            else:
                full[key] = value

    merge_model(state_dict_rank0["model"], state_dict_local["model"])
    if "optimizer" in state_dict_local and "optimizer" in state_dict_rank0:
        full = state_dict_rank0["optimizer"]["optimizer"] if fp16 else state_dict_rank0["optimizer"]
        shard = state_dict_local["optimizer"]["optimizer"] if fp16 else state_dict_local["optimizer"]
        for key, value in shard["state"].items():
            full["state"][key] = value
        if fp16:
            for gi, group in enumerate(state_dict_local["optimizer"]["fp32_from_fp16_params"]):
                for pi, param in enumerate(group):
                    if param is not None:
                        state_dict_rank0["optimizer"]["fp32_from_fp16_params"][gi][pi] = param
    return state_dict_rank0


def _read_tracker(load_dir):
    from megatron.checkpointing import get_checkpoint_tracker_filename
    tracker = get_checkpoint_tracker_filename(load_dir)
    if not os.path.isfile(tracker):
        return None, False
    with open(tracker, "r") as f:
        meta = f.read().strip()
    try:
        return int(meta), False
    except ValueError:
        if meta != "release":
            raise RuntimeError("invalid checkpoint tracker file %s" % tracker)
        return 0, True


def load_checkpoint(model, optimizer, lr_scheduler, load_arg="load"):
    r"""Load a checkpoint written by :func:`save_checkpoint`; returns the iteration."""
    from megatron import get_args, mpu, print_rank_last
    if mpu.get_data_parallel_rank() == 0:
        from megatron.checkpointing import load_checkpoint as load_native
        return load_native(model, optimizer, lr_scheduler, load_arg)

    args = get_args()
    load_dir = getattr(args, load_arg)
    model = _unwrap(model)
    iteration, release = _read_tracker(load_dir)
    if iteration is None:
        print_rank_last("WARNING: no checkpoint tracker in {}: starting from random".format(load_dir))
        return 0
    assert iteration > 0 or release

    name0 = get_fmoe_checkpoint_name(load_dir, iteration, release, 0)
    name_local = get_fmoe_checkpoint_name(load_dir, iteration, release, mpu.get_data_parallel_rank())
    state0 = torch.load(name0, map_location="cpu", weights_only=False)
    state_local = torch.load(name_local, map_location="cpu", weights_only=False)
    state = merge_state_dict(state0, state_local, args.fp16)

    try:
        from megatron.checkpointing import set_checkpoint_version
        set_checkpoint_version(state.get("checkpoint_version", 0))
    except ImportError:
        pass

    if args.finetune or release:
        iteration = 0
    else:
        iteration = state.get("iteration", state.get("total_iters", iteration))

    if "args" in state:
        ckpt_args = state["args"]
        try:
            from megatron.checkpointing import check_checkpoint_args, update_num_microbatches
            check_checkpoint_args(ckpt_args)
            args.consumed_train_samples = getattr(ckpt_args, "consumed_train_samples", 0)
            update_num_microbatches(consumed_samples=args.consumed_train_samples)
            args.consumed_valid_samples = getattr(ckpt_args, "consumed_valid_samples", 0)
        except ImportError:
            pass

    assert len(model) == 1, "interleaved pipelining is not supported (len(model) must be 1)"
    model[0].load_state_dict(state["model"])

    if not release and not args.finetune and not args.no_load_optim:
        if optimizer is not None and "optimizer" in state:
            optimizer.load_state_dict(state["optimizer"])
        if lr_scheduler is not None and "lr_scheduler" in state:
            lr_scheduler.load_state_dict(state["lr_scheduler"])

    if not release and not args.finetune and not args.no_load_rng and "random_rng_state" in state:
        random.setstate(state["random_rng_state"])
        np.random.set_state(state["np_rng_state"])
        torch.set_rng_state(state["torch_rng_state"])
        if torch.cuda.is_available() and "cuda_rng_state" in state:
            torch.cuda.set_rng_state(state["cuda_rng_state"])
        if "rng_tracker_states" in state and hasattr(mpu, "get_cuda_rng_tracker"):
            mpu.get_cuda_rng_tracker().set_states(state["rng_tracker_states"])

    torch.distributed.barrier()
    print_rank_last("  successfully loaded checkpoint (with expert parameters updated) from {} "
                    "at iteration {}".format(load_dir, iteration))
    return iteration
