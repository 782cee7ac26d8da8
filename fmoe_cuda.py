r"""
``import fmoe_cuda`` — the reference's native module name (``cuda/fmoe_cuda.cpp:104-125``).

The thirteen entry points keep their names and argument orders; CUDA tensors run the sm_100a
kernels, CPU tensors the C++/PyTorch CPU ops.  ``ensure_nccl`` records the expert-parallel group
(no private communicator is created); ``smart_sch_forward`` / ``smart_sch_backward`` /
``reduce_grad`` take the reference's callbacks and run the group-wise pipelined schedule with
shadow experts (:mod:`fastmoe_b200.fastermoe.native_api`).
"""
from fastmoe_b200.fastermoe.native_api import reduce_grad, smart_sch_backward, smart_sch_forward  # noqa: F401
from fastmoe_b200.ops.api import (assign_pos, ensure_nccl, expert_count, expert_exchange,  # noqa: F401
                                  global_gather, global_scatter, limit_by_capacity,
                                  linear_backward, linear_forward, prune_gate_by_capacity,
                                  swipe_once)
