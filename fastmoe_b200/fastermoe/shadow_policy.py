r"""
Which experts to shadow (replicate on every rank for one iteration).

Parity: ``fmoe/fastermoe/shadow_policy.py`` — ``global_policy`` (``:10-60``),
``no_shadow_policy`` (``:63-65``), ``get_shadow_policy`` (``:68-73``) and the tuning variables
``FMOE_FASTER_GLBPLC_{NETBW,GPUTP,ALPHA,DMODEL}``.  The performance model is the paper's:
with ``B_w`` the load of the busiest remaining expert, one layer costs about

    3 · T_comp · B_w + 4 · T_feat · B_w + Σ T_model(shadowed)

with ``T_comp = 4·α·d² / bw_mm``, ``T_feat = d·s / bw_net``, ``T_model = 2·α·d²·s / bw_net``
(``s`` = bytes per element).  Experts are shadowed greedily, hottest first, while that lowers
the estimate.  Defaults describe a B200 box (NVLink 5, tcgen05 bf16) instead of the
reference's InfiniBand/V100 numbers, and ``s`` follows the layer's dtype instead of being
fixed at 4.
"""
import os

import torch
import torch.distributed as dist

from .. import config
from ..parallel.comm import get_moe_group

_dtype_bytes = 2


def set_element_size(nbytes):
    global _dtype_bytes
    _dtype_bytes = int(nbytes)


def shadow_plan(expert_loads, d_model, alpha, bw_net, bw_mm, data_size):
    r"""Pure function: bool list over experts (``expert_loads[g]`` tokens for global expert g)."""
    loads = [float(v) for v in expert_loads]
    order = sorted(range(len(loads)), key=lambda g: -loads[g])
    alpha_h2 = alpha * d_model * d_model
    t_feat = d_model * data_size / bw_net
    t_model = 2 * alpha_h2 * data_size / bw_net
    t_comp = 4 * alpha_h2 / bw_mm
    best = 3 * t_comp * loads[order[0]] + 4 * t_feat * loads[order[0]]
    chosen = [False] * len(loads)
    shadow_cost = 0.0
    for i, g in enumerate(order[:-1]):
        nxt = loads[order[i + 1]]
        shadow_cost += t_model
        estimate = 3 * t_comp * nxt + 4 * t_feat * nxt + shadow_cost
        if estimate >= best:
            break
        best = estimate
        chosen[g] = True
    return chosen


def global_policy(local_expert_count, _gec, num_expert, world_size, device):
    r"""Reference signature; returns a CPU bool tensor ``[world_size * num_expert]``."""
    bw_net = config.float_from_env("FMOE_FASTER_GLBPLC_NETBW", config.B200_NVLINK_BYTES_PER_S)
    bw_mm = config.float_from_env("FMOE_FASTER_GLBPLC_GPUTP", config.B200_GEMM_FLOPS)
    alpha = config.float_from_env("FMOE_FASTER_GLBPLC_ALPHA", 2)
    d_model = config.float_from_env("FMOE_FASTER_GLBPLC_DMODEL", 2048)

    lec = local_expert_count.to(device)
    if world_size > 1:
        parts = [torch.empty_like(lec) for _ in range(world_size)]
        dist.all_gather(parts, lec, group=get_moe_group())
        loads = torch.stack(parts).sum(0).cpu()
    else:
        loads = lec.cpu()
    plan = shadow_plan(loads.tolist(), d_model, alpha, bw_net, bw_mm, _dtype_bytes)
    return torch.tensor(plan, dtype=torch.bool)


def no_shadow_policy(_lec, _gec, num_expert, world_size, device):
    return torch.zeros(world_size * num_expert, dtype=torch.bool)


def get_shadow_policy(d_model=None):
    if d_model is not None and "FMOE_FASTER_GLBPLC_DMODEL" not in os.environ:
        os.environ["FMOE_FASTER_GLBPLC_DMODEL"] = str(d_model)
    if not config.switch_from_env("FMOE_FASTER_SHADOW_ENABLE"):
        return no_shadow_policy
    return global_policy
