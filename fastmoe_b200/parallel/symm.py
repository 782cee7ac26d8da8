r"""Symmetric-memory rendezvous and the kernels that run over it (see the module body)."""


def allreduce_grads(grads, comm, scale, fp32_accumulate):  # pylint: disable=unused-argument
    return False
