r"""
Autograd glue of the general MoE path (arbitrary expert modules, pytree inputs).

Public names and argument orders follow ``fmoe/functions.py`` so that user code written
against the reference keeps working: ``count_by_gate`` (``:28-49``), ``prepare_forward``
(``:52-75``), ``MOEScatter`` (``:93-142``), ``MOEGather`` (``:144-193``), ``AllGather``
(``:196-213``), ``Slice`` (``:216-238``), ``ensure_comm`` / ``get_moe_group`` (``:16-25``).

This path needs the per-expert row counts on the host because user experts are called
with Python slices; it therefore keeps exactly one device→host read per layer (the
reference has two plus three ``.cpu()`` copies).  ``FMoETransformerMLP``-shaped experts
never come here on a GPU: they take the fused path in :mod:`fastmoe_b200.ops.fused`,
which has no host read at all.
"""
import torch
import torch.distributed as dist
from torch.autograd import Function

from .ops import api as _ops
from .parallel.comm import ensure_comm, get_moe_group  # noqa: F401  (re-exported)


def count_by_gate(gate, num_expert, world_size, require_pos=True):
    r"""Routing summary ``(pos, local_expert_count, global_expert_count)``.

    ``pos`` lists the kept slots grouped by ascending global expert id (ascending slot id
    inside a group); the counts are int64 tensors on the device of ``gate``.
    """
    with torch.no_grad():
        tot = num_expert * world_size
        counts, rank = _ops.route(gate, tot)
        local_expert_count = counts.long()
        if world_size > 1:
            global_expert_count = _ops.expert_exchange(local_expert_count, num_expert, world_size)
        else:
            global_expert_count = local_expert_count
        if not require_pos:
            return None, local_expert_count, global_expert_count
        flat = gate.reshape(-1)
        starts = torch.cumsum(local_expert_count, 0) - local_expert_count
        kept = flat >= 0
        dest = starts[flat.clamp(min=0)] + rank.long()
        slots = torch.arange(flat.numel(), device=flat.device)
        # Boolean indexing sizes its result from device data: this is the one host read of
        # the general path, shared with the counts copy below in `prepare_forward`.
        pos = torch.empty(int(kept.sum()), dtype=torch.long, device=flat.device)
        pos[dest[kept]] = slots[kept]
    return pos, local_expert_count, global_expert_count


def prepare_forward(gate, num_expert, world_size):
    r"""``(pos, lec_cpu, gec_cpu, fwd_expert_count_cpu, fwd_batch_size)`` for one layer call."""
    pos, lec, gec = count_by_gate(gate, num_expert, world_size)
    with torch.no_grad():
        both = torch.stack([lec, gec]).cpu()
        lec_cpu, gec_cpu = both[0], both[1]
        fwd_expert_count = gec_cpu.view(world_size, num_expert).sum(dim=0)
        fwd_batch_size = int(fwd_expert_count.sum())
    return pos, lec_cpu, gec_cpu, fwd_expert_count, fwd_batch_size


def _local_scatter(inp, pos):
    return torch.index_select(inp, 0, pos)


def _local_gather(inp, pos, out_batch_size, maybe_overlap=True):
    out = torch.zeros((out_batch_size,) + tuple(inp.shape[1:]), dtype=inp.dtype, device=inp.device)
    if maybe_overlap:
        out.index_add_(0, pos, inp)
    else:
        out.index_copy_(0, pos, inp)
    return out


class MOEScatter(Function):
    r"""Rows of ``inp`` → contiguous per-expert segments on the owning ranks."""

    @staticmethod
    def forward(ctx, inp, pos, local_expert_count, global_expert_count, fwd_batch_size, world_size):
        buf = _local_scatter(inp, pos)
        if world_size > 1:
            buf = _ops.global_scatter(buf, local_expert_count, global_expert_count,
                                      fwd_batch_size, world_size)
        ctx.moe_args = inp.shape[0], pos.shape[0], world_size
        ctx.save_for_backward(pos, local_expert_count, global_expert_count)
        return buf

    @staticmethod
    def backward(ctx, grad):
        pos, lec, gec = ctx.saved_tensors
        inp_batch, buf_batch, world_size = ctx.moe_args
        grad = grad.contiguous()
        if world_size > 1:
            grad = _ops.global_gather(grad, lec, gec, buf_batch, world_size)
        return _local_gather(grad, pos, inp_batch), None, None, None, None, None


class MOEGather(Function):
    r"""Expert outputs → ``[local_batch_size, d]`` rows in slot order (dropped slots stay zero)."""

    @staticmethod
    def forward(ctx, global_output_buf, pos, local_expert_count, global_expert_count,
                local_batch_size, world_size):
        buf = global_output_buf.contiguous()
        if world_size > 1:
            buf = _ops.global_gather(buf, local_expert_count, global_expert_count,
                                     pos.shape[0], world_size)
        out = _local_gather(buf, pos, local_batch_size, maybe_overlap=False)
        ctx.moe_args = global_output_buf.shape[0], world_size
        ctx.save_for_backward(pos, local_expert_count, global_expert_count)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        pos, lec, gec = ctx.saved_tensors
        fwd_batch_size, world_size = ctx.moe_args
        buf = _local_scatter(grad_out.contiguous(), pos)
        if world_size > 1:
            buf = _ops.global_scatter(buf, lec, gec, fwd_batch_size, world_size)
        return buf, None, None, None, None, None


class AllGather(Function):
    r"""Differentiable all-gather along dim 0 (backward keeps this rank's slice)."""

    @staticmethod
    def forward(ctx, inp, rank, world_size, group):
        inp = inp.contiguous()
        out = _p2p_allgather(inp, group)
        if out is None:
            out = inp.new_empty((world_size * inp.shape[0],) + tuple(inp.shape[1:]))
            if inp.is_cuda:
                dist.all_gather_into_tensor(out, inp, group=group)
            else:
                _all_gather_cat(out, inp, world_size, group)
        ctx.args = rank, inp.shape[0]
        return out

    @staticmethod
    def backward(ctx, grad_out):
        rank, n = ctx.args
        return grad_out[rank * n:(rank + 1) * n], None, None, None


def _p2p_allgather(inp, group, out=None):
    r"""Peer-to-peer all-gather on GPUs with a symmetric workspace, else ``None``."""
    if not inp.is_cuda:
        return None
    from .parallel import symm
    return symm.allgather_rows(inp, group, out)


def _all_gather_cat(out, inp, world_size, group):
    parts = list(out.chunk(world_size, dim=0))
    dist.all_gather(parts, inp, group=group)


class Slice(Function):
    r"""Keep rows ``[rank*B//W, (rank+1)*B//W)``; backward all-gathers the gradient slices.

    As in the reference the remainder rows ``B % W`` are not routed.
    """

    @staticmethod
    def forward(ctx, inp, rank, world_size, group):
        n = inp.shape[0] // world_size
        ctx.args = world_size, group, inp.shape[0]
        return inp[n * rank:min(n * (rank + 1), inp.shape[0])]

    @staticmethod
    def backward(ctx, grad_out):
        world_size, group, full = ctx.args
        grad_out = grad_out.contiguous()
        out = grad_out.new_zeros((full,) + tuple(grad_out.shape[1:]))
        covered = out[:world_size * grad_out.shape[0]]
        if _p2p_allgather(grad_out, group, out=covered) is not None:
            pass
        elif grad_out.is_cuda:
            dist.all_gather_into_tensor(covered, grad_out, group=group)
        else:
            _all_gather_cat(covered, grad_out, world_size, group)
        return out, None, None, None
