r"""
Collective-library transport for the *general* MoE path.

This is the comparison path (``FMOE_FUSED=0``) and the path used by arbitrary expert
modules, CPU tensors and ``gloo`` ranks: the variable-size all-to-all of token rows is a
single ``all_to_all_single`` with split sizes instead of the reference's host loop of one
``ncclSend/ncclRecv`` per (expert, peer) (``cuda/global_exchange.h:28-53,73-98``).  The
buffer layouts are the reference's: rows leave ordered by global expert id (destination
rank outer, local expert inner) and arrive ordered local expert outer, source rank inner.

The product path for ``FMoETransformerMLP``-shaped experts on B200 does not come through
here: it uses the peer-to-peer kernels in :mod:`fastmoe_b200.ops.fused`.
"""
import torch
import torch.distributed as dist

_moe_group = None


def get_torch_default_comm():
    r"""The default process group (parity: ``fmoe/utils.py:10-31``)."""
    try:
        return dist.distributed_c10d._get_default_group()  # pylint: disable=protected-access
    except Exception as exc:  # pylint: disable=broad-except
        raise RuntimeError("torch.distributed is not initialised") from exc


def get_rank_0_in_comm(comm):
    r"""Global rank of the member with group-rank 0 (parity: ``fmoe/utils.py:34-40``), without a collective."""
    return dist.get_global_rank(comm, 0) if comm is not None else 0


def set_moe_group(comm):
    global _moe_group
    _moe_group = comm


def get_moe_group():
    return _moe_group


def ensure_comm(t, comm):
    r"""Record the expert-parallel group used by the exchange ops (parity: ``fmoe/functions.py:16-21``).

    The reference builds a private NCCL communicator here; nothing of the sort is needed:
    the general path uses the group's own collectives and the fused path a symmetric-memory
    rendezvous on the same group.
    """
    if comm is None:
        comm = get_torch_default_comm()
    set_moe_group(comm)


def _group(group):
    return group if group is not None else _moe_group


def expert_exchange(local_expert_count, n_expert, n_worker, group=None):
    r"""All-to-all of ``n_expert`` counts per peer (parity: ``cuda/global_exchange.cpp:9-46``)."""
    out = torch.empty_like(local_expert_count)
    dist.all_to_all_single(out, local_expert_count.contiguous(), group=_group(group))
    return out


def _recv_permutation(gec_cpu, n_expert, n_worker):
    r"""Index that reorders rows received source-major into expert-major/source-minor order."""
    cnt = gec_cpu.view(n_worker, n_expert)
    src_major_start = torch.cumsum(cnt.reshape(-1), 0) - cnt.reshape(-1)
    pieces = []
    for e in range(n_expert):
        for w in range(n_worker):
            n = int(cnt[w, e])
            if n:
                s = int(src_major_start[w * n_expert + e])
                pieces.append(torch.arange(s, s + n))
    if not pieces:
        return torch.empty(0, dtype=torch.int64)
    return torch.cat(pieces)


def global_scatter(local_input_buf, lec_cpu, gec_cpu, batch_size, n_worker, group=None):
    r"""Send rows grouped by global expert to their owners (parity: ``cuda/global_exchange.h:11-55``)."""
    n_expert = lec_cpu.numel() // n_worker
    send = lec_cpu.view(n_worker, n_expert).sum(1).tolist()
    recv = gec_cpu.view(n_worker, n_expert).sum(1).tolist()
    out = local_input_buf.new_empty((batch_size,) + tuple(local_input_buf.shape[1:]))
    dist.all_to_all_single(out, local_input_buf.contiguous(), recv, send, group=_group(group))
    if n_expert > 1 and batch_size > 0:
        perm = _recv_permutation(gec_cpu, n_expert, n_worker).to(out.device)
        out = out.index_select(0, perm)
    return out


def global_gather(global_output_buf, lec_cpu, gec_cpu, batch_size, n_worker, group=None):
    r"""Inverse of :func:`global_scatter` (parity: ``cuda/global_exchange.h:57-100``)."""
    n_expert = lec_cpu.numel() // n_worker
    send = gec_cpu.view(n_worker, n_expert).sum(1).tolist()
    recv = lec_cpu.view(n_worker, n_expert).sum(1).tolist()
    buf = global_output_buf
    if n_expert > 1 and buf.shape[0] > 0:
        perm = _recv_permutation(gec_cpu, n_expert, n_worker).to(buf.device)
        src_major = torch.empty_like(buf)
        src_major.index_copy_(0, perm, buf)
        buf = src_major
    out = buf.new_empty((batch_size,) + tuple(buf.shape[1:]))
    dist.all_to_all_single(out, buf.contiguous(), recv, send, group=_group(group))
    return out
