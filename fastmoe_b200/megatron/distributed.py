r"""Megatron-facing DDP wrapper (parity: ``fmoe/megatron/distributed.py:12-77``)."""
import torch

from ..distributed import DistributedGroupedDataParallel

_groups = None


def _set_groups(**kwargs):
    global _groups
    _groups = kwargs


def get_moe_group():
    return _groups["moe_group"]


def _init():
    r"""``gate_group`` = all ranks of one pipeline stage (gates are replicated inside a stage);
    ``dp_group`` = ``moe_group`` = Megatron's data-parallel group."""
    from megatron import get_args, mpu
    args = get_args()
    stage_size = args.world_size // args.pipeline_model_parallel_size
    gate_group = None
    for first in range(0, args.world_size, stage_size):
        ranks = list(range(first, first + stage_size))
        group = torch.distributed.new_group(ranks)
        if args.rank in ranks:
            gate_group = group
    _set_groups(dp_group=mpu.get_data_parallel_group(), moe_group=mpu.get_data_parallel_group(),
                gate_group=gate_group)


class DistributedDataParallel(DistributedGroupedDataParallel):
    r"""Replacement of Megatron's ``LocalDDP``: gradients are reduced per ``dp_comm`` tag."""

    def __init__(self, module, accumulate_allreduce_grads_in_fp32=False,
                 use_contiguous_buffers_in_ddp=False):
        assert not accumulate_allreduce_grads_in_fp32, \
            "accumulate_allreduce_grads_in_fp32 is not supported"
        assert not use_contiguous_buffers_in_ddp, "use_contiguous_buffers_in_ddp is not supported"
        if _groups is None:
            _init()
        super().__init__(module, **_groups)

    # Megatron's module API is forwarded to the wrapped model.
    def set_input_tensor(self, *args, **kwargs):
        return self.module.set_input_tensor(*args, **kwargs)

    def state_dict(self, *args, **kwargs):
        return self.module.state_dict(*args, **kwargs)

    def state_dict_for_save_checkpoint(self, *args, **kwargs):
        return self.module.state_dict_for_save_checkpoint(*args, **kwargs)

    def load_state_dict(self, *args, **kwargs):
        return self.module.load_state_dict(*args, **kwargs)
