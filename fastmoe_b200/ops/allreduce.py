r"""Fused gradient all-reduce entry (filled by the symmetric-memory kernels when available)."""


def try_fused_allreduce(grads, comm, scale, fp32_accumulate=False):  # pylint: disable=unused-argument
    r"""Reduce ``grads`` in place over ``comm`` with the peer-to-peer kernel.

    Returns ``False`` when the tensors are not on a GPU or the group has no symmetric-memory
    rendezvous, in which case the caller uses the collective library.
    """
    if not grads or not grads[0].is_cuda:
        return False
    from ..parallel import symm
    return symm.allreduce_grads(grads, comm, scale, fp32_accumulate)
