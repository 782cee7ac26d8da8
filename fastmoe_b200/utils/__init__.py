r"""Helpers: pytree mapping, process-group lookup (``fmoe/utils.py``), timers and logging."""
from ..parallel.comm import get_rank_0_in_comm, get_torch_default_comm  # noqa: F401


def check_device_status(device=None, clear=True):
    r"""Raise if a kernel of this library reported a failure on ``device`` since the last check.

    Kernels never trap: a bounded wait that ran out (a peer that never arrived) or a receive
    buffer that overflowed leaves a code in a per-device status word and the kernel returns.
    Reading the word synchronises the device, so call this at logging or checkpoint intervals,
    not every step.
    """
    import torch
    from ..ops import native
    if not torch.cuda.is_available() or not native.available():
        return 0
    nat = native.get()
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    code = int(nat.read_status(index))
    if code != 0:
        if clear:
            nat.clear_status(index)
        names = {nat.STATUS_PEER_TIMEOUT: "a peer did not arrive within FMOE_WAIT_TIMEOUT_MS",
                 nat.STATUS_RECV_OVERFLOW: "more rows were routed to a rank than FMOE_RECV_CAPACITY_FACTOR allows",
                 101: "grouped GEMM producer wait timed out", 102: "grouped GEMM MMA wait timed out",
                 103: "grouped GEMM epilogue wait timed out"}
        raise RuntimeError("fastmoe_b200 device status %d on cuda:%d: %s"
                           % (code, index, names.get(code, "unknown failure")))
    return 0
