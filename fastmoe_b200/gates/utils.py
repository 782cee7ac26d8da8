r"""Capacity helper shared by the balanced gates (parity: ``fmoe/gates/utils.py:9-26``)."""
import torch

from ..functions import count_by_gate
from ..ops import api as _ops


def limit_by_capacity(topk_idx, num_expert, world_size, capacity, group=None):
    r"""Enforce a per-local-expert ``capacity`` across all ranks.

    Every expert owner grants its capacity to the requesting ranks in rank order; ranks then
    drop the slots beyond their grant (slot order).  Returns ``(new_lec, new_gec, topk_idx)``.
    ``group`` is the expert-parallel group of the layer the gate belongs to (default: the group
    the layer recorded with ``ensure_comm``, else all processes).
    """
    with torch.no_grad():
        cap = torch.full((num_expert,), int(capacity), dtype=torch.int32, device=topk_idx.device)
        if world_size > 1 and topk_idx.is_cuda:
            # One peer-to-peer exchange of requests and capacities; every rank derives all
            # grants from the full matrix, so nothing has to travel back.
            from ..parallel import comm as _comm, symm as _symm
            counts, _rank = _ops.route(topk_idx, num_expert * world_size)
            fused = _symm.capacity_grant(counts, cap, num_expert, _comm._group(group))  # pylint: disable=protected-access
            if fused is not None:
                new_lec, new_gec = fused
                topk_idx = _ops.prune_gate_by_capacity(
                    topk_idx, new_lec.to(torch.int32), num_expert, world_size)
                return new_lec, new_gec, topk_idx
        _, _lec, gec = count_by_gate(topk_idx, num_expert, world_size, require_pos=False)
        new_gec = _ops.limit_by_capacity(gec, cap, num_expert, world_size)
        if world_size > 1:
            new_lec = _ops.expert_exchange(new_gec, num_expert, world_size, group=group)
        else:
            new_lec = new_gec
        topk_idx = _ops.prune_gate_by_capacity(
            topk_idx, new_lec.to(torch.int32), num_expert, world_size)
    return new_lec, new_gec, topk_idx
