r"""
Shadow experts on the fused expert-parallel path of ``FMoETransformerMLP``.

FasterMoE replicates ("shadows") the hottest experts on every rank for one iteration, so that
their tokens need not travel at all (``cuda/fastermoe/smart_schedule.h:106-261``: the native
scheduler broadcasts the parameters, runs the shadowed expert locally on the rank's own rows,
and reduces its gradients to the owner in backward).  Here the same thing is composed from the
kernels of the product path, without leaving the fused path:

* the shadow policy (``shadow_policy.py``) decides which global experts are shadowed;
* slots routed to a shadowed expert are masked out of the expert-parallel call — the fused
  dispatch / GEMM / combine kernels skip dropped slots, so nothing of them crosses NVLink;
* the owner of every shadowed expert pushes its parameters to all ranks with the peer-to-peer
  broadcast kernel (one write per peer);
* the masked slots run through the single-GPU fused path (scatter, grouped GEMMs with the fused
  activation, combine) with the shadowed experts as its groups;
* the two partial outputs are added; autograd runs the mirror image, and the backward of the
  parameter broadcast is the reduce-to-owner kernel.

The policy needs the global expert loads on the host, so a layer call with shadowing enabled
contains one host synchronisation (as every call of the reference does) and cannot be captured
in a CUDA graph.
"""
import torch
import torch.distributed as dist

from ..ops import fused
from . import expert_utils
from .schedule import _BroadcastParams
from .shadow_policy import get_shadow_policy, set_element_size

_policy = None


def shadow_mask(layer, idx, x):
    r"""CPU bool tensor over global experts: which ones are shadowed in this call."""
    global _policy
    from ..ops import native
    if _policy is None:
        _policy = get_shadow_policy(d_model=x.shape[-1])
    set_element_size(x.element_size())
    tot = layer.num_expert * layer.world_size
    lec, _rank = native.get().route(idx.reshape(-1).contiguous(), tot)
    return _policy(lec.long(), None, layer.num_expert, layer.world_size, x.device)


def moe_mlp_forward(layer, x, gate_idx, gate_score, stored=None):
    r"""``FMoETransformerMLP`` forward with shadow experts; ``stored`` (bool ``[tot]``) overrides
    the policy.  Falls back to the plain fused path when nothing is shadowed."""
    from ..parallel.symm import _layer_group
    tot = layer.num_expert * layer.world_size
    if stored is None:
        stored = shadow_mask(layer, gate_idx, x)
    stored = stored.reshape(-1).to(torch.bool).cpu()
    shadow_ids = [g for g in range(tot) if bool(stored[g])]
    if not shadow_ids or layer.world_size == 1:
        return fused.moe_mlp_forward(layer, x, gate_idx, gate_score)

    group = _layer_group(layer)
    me = dist.get_rank(group)
    dev = x.device
    stored_dev = stored.to(dev)
    remap = torch.full((tot,), -1, dtype=torch.long)
    remap[shadow_ids] = torch.arange(len(shadow_ids))
    remap = remap.to(dev)
    safe = gate_idx.clamp_min(0)
    is_shadow = stored_dev[safe] & (gate_idx >= 0)
    minus = torch.full_like(gate_idx, -1)
    idx_ep = torch.where(is_shadow, minus, gate_idx)
    idx_local = torch.where(is_shadow, remap[safe], minus)

    out = fused.moe_mlp_forward(layer, x, idx_ep, gate_score)

    experts = layer.experts
    size = expert_utils.get_expert_param_size(experts, 0)
    ref = experts.htoh4.weight
    anchor = torch.zeros(0, device=dev, requires_grad=torch.is_grad_enabled())
    parts = []
    for g in shadow_ids:
        owner, e = divmod(g, layer.num_expert)
        if owner == me:
            flat = expert_utils.flat_expert_params(experts, e)
        else:
            flat = torch.zeros(size, dtype=ref.dtype, device=dev)
        owner_global = dist.get_global_rank(group, owner)
        flat = _BroadcastParams.apply(flat, anchor, owner_global, owner == me, group)
        parts.append(expert_utils.unflatten_like(experts, flat, 0))
    w1 = torch.stack([p[0] for p in parts])
    b1 = torch.stack([p[1] for p in parts])
    w2 = torch.stack([p[2] for p in parts])
    b2 = torch.stack([p[3] for p in parts])
    local = fused.moe_mlp_local(x, idx_local, gate_score, w1, b1, w2, b2, experts.activation)
    return out + local
