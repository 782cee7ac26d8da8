r"""
Device dispatch of the native ops.

The functions here carry the names and argument conventions of the reference's pybind
entry points (``cuda/fmoe_cuda.cpp:104-125``) so that :mod:`fastmoe_b200.fmoe_cuda` can
re-export them one to one.  CUDA tensors run the sm_100a kernels of the extension
(missing extension = error); CPU tensors run the C++ CPU ops of the extension or, when it
is not built, the PyTorch restatement.
"""
import torch

from . import native, torch_impl
from ..parallel import comm as _comm


def _tot(n_expert, n_worker):
    return int(n_expert) * int(n_worker)


# ------------------------------------------------------------------ routing bookkeeping
def expert_count(gate_idx, expert_count_out):
    r"""In-place histogram, ``-1`` skipped.  ``expert_count_out`` is int32 ``[tot_expert]``."""
    tot = expert_count_out.numel()
    if gate_idx.is_cuda:
        native.get().expert_count(gate_idx.contiguous().view(-1), expert_count_out)
    else:
        expert_count_out.add_(torch_impl.expert_count(gate_idx, tot))
    return expert_count_out


def assign_pos(cum_count, gate_idx, pos):
    r"""Fill ``pos`` (int64, length ``cum_count[-1]``) with slot ids grouped by expert.

    ``cum_count`` is the inclusive prefix sum of the counts (int32).  Unlike the reference
    kernel (``cuda/local_exchange.cuh:5-16``) it is not consumed, and the order inside an
    expert is ascending slot id.
    """
    tot = cum_count.numel()
    if gate_idx.is_cuda:
        native.get().assign_pos(cum_count, gate_idx.contiguous().view(-1), pos)
    else:
        pos.copy_(torch_impl.assign_pos(gate_idx, tot))
    return pos


def route(gate_idx, tot_expert):
    r"""One-pass routing summary: ``(counts int32[tot], slot_rank int32[n_slots])``.

    ``slot_rank`` is the rank of a slot among the slots of the same expert (``-1`` when the
    slot is dropped) — the quantity the fused dispatch needs instead of ``pos``.
    """
    if gate_idx.is_cuda:
        return native.get().route(gate_idx.contiguous().view(-1), int(tot_expert))
    cnt = torch_impl.expert_count(gate_idx, tot_expert)
    rank = torch_impl.slot_rank(gate_idx, tot_expert).reshape(-1).to(torch.int32)
    return cnt, rank


def limit_by_capacity(expert_count_w, capacity, n_expert, n_worker):
    if expert_count_w.is_cuda:
        return native.get().limit_by_capacity(expert_count_w, capacity, int(n_expert), int(n_worker))
    return torch_impl.limit_by_capacity(expert_count_w, capacity, n_expert, n_worker)


def prune_gate_by_capacity(gate_idx, expert_count_cap, n_expert, n_worker):
    if gate_idx.is_cuda:
        return native.get().prune_gate_by_capacity(
            gate_idx.contiguous(), expert_count_cap, int(n_expert), int(n_worker))
    return torch_impl.prune_gate_by_capacity(gate_idx, expert_count_cap, n_expert, n_worker)


# ------------------------------------------------------------------ grouped linear
_TC_DTYPES = (torch.bfloat16, torch.float16)


def linear_forward(inp, expert_count_cpu, weight, bias=None):
    r"""Grouped linear forward with host-resident counts (the reference's calling convention)."""
    if inp.is_cuda:
        from . import grouped_gemm
        return grouped_gemm.linear_forward_host_counts(inp, expert_count_cpu, weight, bias)
    return torch_impl.linear_forward(inp, expert_count_cpu, weight, bias)


def linear_backward(grad_out, inp, expert_count_cpu, weight, bias=None):
    if inp.is_cuda:
        from . import grouped_gemm
        return grouped_gemm.linear_backward_host_counts(grad_out, inp, expert_count_cpu, weight, bias)
    return torch_impl.linear_backward(grad_out, inp, expert_count_cpu, weight, bias)


# ------------------------------------------------------------------ exchange (general path)
expert_exchange = _comm.expert_exchange
global_scatter = _comm.global_scatter
global_gather = _comm.global_gather


def ensure_nccl(comm, _tensor=None):
    _comm.ensure_comm(_tensor, comm)


# ------------------------------------------------------------------ SWIPE
def swipe_once(gate_idx, capacity, n_expert, n_worker, bias, group=None):
    r"""One SWIPE round (parity: ``cuda/balancing.cu:83-186``): returns ``(new_idx_cpu, capacity_left)``.

    The reference does two count exchanges, an all-reduce and an all-gather with a host
    sync after each.  On B200s one kernel exchanges the request counts and capacities through
    the symmetric heap and computes the plan on every rank, and two small kernels rewrite the
    ids: no host read at all (``parallel/symm.py::swipe_round``).  Elsewhere (CPU tensors,
    ``gloo``): one all-gather gives every rank the whole picture and the plan is computed
    redundantly on the host.
    """
    import torch.distributed as dist
    group = group if group is not None else _comm.get_moe_group()
    idx = gate_idx.reshape(-1)
    if idx.is_cuda and n_worker > 1 and torch.is_tensor(capacity):
        # B200 path: count exchange, plan and reassignment as kernels over the symmetric heap,
        # nothing read on the host (results stay on the device)
        from ..parallel import symm as _symm
        done = _symm.swipe_round(idx, capacity, n_expert, n_worker, bias, group)
        if done is not None:
            return done[0].view_as(gate_idx), done[1]
    worker = torch.div(idx, n_expert, rounding_mode="floor")
    mine = torch.bincount(worker, minlength=n_worker)[:n_worker].to(torch.int64)
    cap = capacity.reshape(1).to(device=idx.device, dtype=torch.int64)
    packed = torch.cat([mine, cap])
    if n_worker > 1:
        gathered = [torch.empty_like(packed) for _ in range(n_worker)]
        dist.all_gather(gathered, packed, group=group)
        rank = dist.get_rank(group)
    else:
        gathered = [packed]
        rank = 0
    table = torch.stack(gathered).cpu()
    accepted, cap_left = torch_impl.swipe_plan(
        table[:, :n_worker].tolist(), table[:, n_worker].tolist(), n_worker)
    new_idx = torch_impl.swipe_reassign(idx, accepted[rank], n_expert, int(bias))
    return new_idx.cpu(), torch.tensor(cap_left[rank], dtype=torch.int64)
