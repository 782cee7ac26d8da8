r"""
``import fmoe_cuda`` — the reference's native module name (``cuda/fmoe_cuda.cpp:104-125``).

The thirteen entry points keep their names and argument orders; CUDA tensors run the sm_100a
kernels, CPU tensors the C++/PyTorch CPU ops.  ``ensure_nccl`` records the expert-parallel group
(no private communicator is created), ``smart_sch_forward`` / ``smart_sch_backward`` /
``reduce_grad`` are superseded by :mod:`fastmoe_b200.fastermoe.schedule`, whose backward is
derived by autograd; they raise with that pointer.
"""
from fastmoe_b200.ops.api import (assign_pos, ensure_nccl, expert_count, expert_exchange,  # noqa: F401
                                  global_gather, global_scatter, limit_by_capacity,
                                  linear_backward, linear_forward, prune_gate_by_capacity,
                                  swipe_once)


def _superseded(name):
    def fn(*_args, **_kwargs):
        raise NotImplementedError(
            "fmoe_cuda.%s is superseded: use fastmoe_b200.fastermoe.schedule.MoEForward / "
            "smart_schedule_forward (autograd derives the backward schedule)" % name)
    fn.__name__ = name
    return fn


smart_sch_forward = _superseded("smart_sch_forward")
smart_sch_backward = _superseded("smart_sch_backward")
reduce_grad = _superseded("reduce_grad")
