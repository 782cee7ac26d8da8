r"""
Gradient-reduction wrapper that replaces Megatron-LM's local DDP.

Parity: ``fmoe/megatron/distributed.py:12-77``.  Three process groups drive the reduction of
the three kinds of parameters of an ``fmoefy``-ed model:

* dense parameters (tag ``'dp'``) and, when experts are replicated, expert parameters: Megatron's
  data-parallel group;
* the expert-parallel exchange (``moe_group``): the same data-parallel group;
* gate parameters (tag ``'gate'``): all ranks of one pipeline stage, i.e. ``world_size /
  pipeline_model_parallel_size`` consecutive ranks.

The groups are created once per process, on first use (creating a group is a collective, so all
ranks construct the wrapper at the same point, as they do in Megatron's ``setup_model``).
"""
import torch.distributed as dist

from ..distributed import DistributedGroupedDataParallel


class _GroupRegistry:
    r"""Lazily built ``{dp_group, moe_group, gate_group}`` of this process."""

    def __init__(self):
        self._groups = None

    def set(self, **groups):
        self._groups = dict(groups)

    def reset(self):
        self._groups = None

    def get(self):
        if self._groups is None:
            self._groups = self._build()
        return self._groups

    @staticmethod
    def _build():
        from megatron import get_args, mpu
        args = get_args()
        per_stage = args.world_size // args.pipeline_model_parallel_size
        gate_group = None
        # every rank takes part in the creation of every stage's group
        for stage in range(args.pipeline_model_parallel_size):
            members = list(range(stage * per_stage, (stage + 1) * per_stage))
            handle = dist.new_group(members)
            if args.rank in members:
                gate_group = handle
        data_parallel = mpu.get_data_parallel_group()
        return dict(dp_group=data_parallel, moe_group=data_parallel, gate_group=gate_group)


_registry = _GroupRegistry()


def _set_groups(**kwargs):
    r"""Install groups explicitly (tests, or programs that manage their own groups)."""
    _registry.set(**kwargs)


def get_moe_group():
    return _registry.get()["moe_group"]


# Methods of the wrapped Megatron module that callers expect to find on the wrapper.
_FORWARDED = ("set_input_tensor", "state_dict", "state_dict_for_save_checkpoint", "load_state_dict")


class DistributedDataParallel(DistributedGroupedDataParallel):
    r"""Drop-in for Megatron's ``LocalDDP``: gradients are reduced per ``dp_comm`` tag in the groups
    above; the model-facing methods Megatron calls on its DDP wrapper go to the wrapped module."""

    def __init__(self, module, accumulate_allreduce_grads_in_fp32=False,
                 use_contiguous_buffers_in_ddp=False):
        if accumulate_allreduce_grads_in_fp32:
            raise AssertionError("accumulate_allreduce_grads_in_fp32 is not supported "
                                 "(pass fp32_allreduce=True to allreduce_gradients instead)")
        if use_contiguous_buffers_in_ddp:
            raise AssertionError("use_contiguous_buffers_in_ddp is not supported")
        super().__init__(module, **_registry.get())


def _forward_to_module(name):
    def method(self, *args, **kwargs):
        return getattr(self.module, name)(*args, **kwargs)
    method.__name__ = name
    method.__doc__ = "Forwarded to the wrapped module (Megatron calls it on the DDP wrapper)."
    return method


for _name in _FORWARDED:
    setattr(DistributedDataParallel, _name, _forward_to_module(_name))
