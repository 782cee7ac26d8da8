r"""
One place for every environment switch of the framework.

The reference scatters its switches over several modules
(``fmoe/fastermoe/config.py:4-13``, ``fmoe/layers.py:81-84``,
``fmoe/fastermoe/shadow_policy.py:19-22,69-71``, ``fmoe/gates/faster_gate.py:26-41``,
``cuda/fastermoe/smart_schedule.cpp:78-86``).  The names and defaults are kept; the
performance-model defaults are re-based to a B200 box (NVLink 5 instead of
InfiniBand, tcgen05 bf16 instead of V100 fp32).  New switches control the fused
sm_100a paths.
"""
import os

_TRUE = ("1", "ON", "on", "true", "True", "TRUE")


def float_from_env(key, default=-1):
    r"""Float value of ``$key``, ``default`` when unset."""
    if key in os.environ:
        return float(os.environ[key])
    return default


def int_from_env(key, default=0):
    r"""Integer value of ``$key``, ``default`` when unset."""
    if key in os.environ:
        return int(os.environ[key])
    return default


def switch_from_env(key, default=False):
    r"""Boolean switch: the reference accepts ``'1'`` and ``'ON'``; a few more spellings are tolerated."""
    if key in os.environ:
        return os.environ[key] in _TRUE
    return default


# ---------------------------------------------------------------------------------
# Reference-compatible switches
# ---------------------------------------------------------------------------------
def faster_schedule_enabled():
    return switch_from_env("FMOE_FASTER_SCHEDULE_ENABLE", False)


def faster_shadow_enabled():
    return switch_from_env("FMOE_FASTER_SHADOW_ENABLE", False)


def faster_group_size(default=4):
    return max(1, int_from_env("FMOE_FASTER_GROUP_SIZE", default))


def topo_gpus_per_node(default=8):
    try:
        return int(os.environ["FMOE_TOPO_GPUS_PER_NODE"])
    except (KeyError, ValueError):
        return default


def topo_outgoing_fraction(default=0.14):
    try:
        return float(os.environ["FMOE_TOPO_OUTGOING_FRACTION"])
    except (KeyError, ValueError):
        return default


# B200 defaults of the shadow-expert performance model: one direction of NVLink 5
# through NVSwitch, and a conservative sustained bf16 tcgen05 GEMM rate.
B200_NVLINK_BYTES_PER_S = 900e9
B200_GEMM_FLOPS = 1.3e15


# ---------------------------------------------------------------------------------
# New switches (fused sm_100a paths)
# ---------------------------------------------------------------------------------
def fused_enabled():
    r"""``FMOE_FUSED=0`` forces the collective-library comparison path for dispatch/combine."""
    return switch_from_env("FMOE_FUSED", True)


def wait_timeout_ms():
    r"""Upper bound of every device-side wait on a peer, in milliseconds.

    Generous by default (a peer may legitimately be late: a checkpoint being written, a
    garbage-collection pause); tests that exercise the time-out path set a few hundred ms.
    """
    return int_from_env("FMOE_WAIT_TIMEOUT_MS", 30000)


def debug_bounds():
    r"""``FMOE_DEBUG_BOUNDS=1``: the fused paths validate the routing tables on the host
    (expert ids in range, slot ranks consistent with the counts, offsets monotone and inside
    the buffers) before launching; costs a device synchronisation per layer call."""
    return switch_from_env("FMOE_DEBUG_BOUNDS", False)


def nvtx_enabled():
    r"""``FMOE_NVTX=1``: NVTX ranges around the fused paths (forward, backward, exchange,
    gradient all-reduce) for timeline tools."""
    return switch_from_env("FMOE_NVTX", False)


def ep_trace():
    r"""``FMOE_EP_TRACE=1``: the fused dispatch + GEMM kernel of the expert-parallel forward
    writes four ``%globaltimer`` stamps per CTA (entry, first rows available, sender done, exit);
    read them with ``utils.profiling.ep_trace_summary()``."""
    return switch_from_env("FMOE_EP_TRACE", False)


def use_nvls():
    r"""``FMOE_USE_NVLS=1``: gradient all-reduce through NVSwitch (``multimem.ld_reduce`` /
    ``multimem.st`` on the multicast mapping of the symmetric buffer) when the allocation has
    one; plain peer loads and stores otherwise.  Off by default: keep it off in runs where a rank
    may leave while its memory is bound to a multicast object (failure tests)."""
    return switch_from_env("FMOE_USE_NVLS", False)


def recv_capacity_factor():
    r"""Rows reserved in the expert receive buffer, as a multiple of the balanced load.

    ``0`` (default) reserves the worst case (every token of every rank lands on one rank),
    which is what 180 GB of HBM per GPU is for; a positive factor bounds the buffer and turns
    overflow into a reported error.
    """
    return float_from_env("FMOE_RECV_CAPACITY_FACTOR", 0.0)


def force_ep_path():
    r"""``FMOE_FORCE_EP=1``: layers with ``world_size == 1`` inside an initialised one-rank NCCL
    group take the expert-parallel kernels (sender warps, arrival flags, return push) instead of
    the single-GPU path.  Every peer table then points at the GPU itself; used to test and
    profile the multi-GPU code on one GPU."""
    return switch_from_env("FMOE_FORCE_EP", False)


def max_tokens():
    r"""``FMOE_MAX_TOKENS``: tokens per rank the exchange buffers of the fused expert-parallel
    path are sized for.  ``0`` (default): the ranks agree on the largest batch of the first call."""
    return int_from_env("FMOE_MAX_TOKENS", 0)


def push_before_wgrad():
    r"""``FMOE_PUSH_BEFORE_WGRAD`` (default off): in the fused expert-parallel backward, queue the
    input-gradient GEMM whose epilogue returns rows to their sources before the two weight
    gradients instead of after them.  The idea is to cover the flight time of the remote stores
    with local GEMMs; measured on 8 B200s it is slower (0.928 against 0.869 ms per step of the
    headline layer: the weight gradients then run while the peers' rows are landing in this
    GPU's memory), on 2 GPUs it makes no difference."""
    return switch_from_env("FMOE_PUSH_BEFORE_WGRAD", False)
