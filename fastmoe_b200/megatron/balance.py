r"""
Balance monitoring for ``fmoefy``-ed Megatron models.

Parity: ``fmoe/megatron/balance.py:11-78`` (``reset_gate_hook``, ``get_balance_profile``,
``generate_megatron_gate_hook``, ``add_balance_log`` and the module-level ``balance_dict`` /
``num_layers``).  Every MoE layer gets a gate hook that feeds one shared profile — per metric a
vector with one entry per layer, see :mod:`fastmoe_b200.balance` — and ``add_balance_log``
averages the layers' balance losses over all ranks and writes TensorBoard scalars
``balance-<metric>/layer-<i>`` and ``balance-<metric>/all``.
"""
import torch
import torch.distributed as dist

from .. import balance as _profile
from ..parallel.comm import get_torch_default_comm

balance_dict = {}      # metric name -> per-layer tensor; shared with the hooks below
num_layers = 0


def _strategy():
    from megatron import get_args
    return get_args().balance_strategy


def reset_gate_hook(_num_layers=None):
    r"""(Re)initialise the shared profile for ``_num_layers`` layers (kept from the last call
    when omitted)."""
    global num_layers
    num_layers = num_layers if _num_layers is None else _num_layers
    _profile.reset_balance_profile(balance_dict, num_layers, _strategy())


def get_balance_profile():
    return balance_dict


def generate_megatron_gate_hook(layer_idx, num_expert_global):
    r"""A ``gate_hook(idx, score, context)`` that records layer ``layer_idx`` into the profile."""
    strategy = _strategy()

    def megatron_gate_hook(gate_top_k_idx, gate_score_top_k, gate_context):
        _profile.update_balance_profile(balance_dict, gate_top_k_idx, gate_score_top_k,
                                        gate_context, layer_idx, num_expert_global, strategy)

    return megatron_gate_hook


def _moe_gates(model):
    r"""Gates of all transformer layers, for every Megatron layout the adapter knows."""
    while hasattr(model, "module"):
        model = model.module
    lm = model.language_model
    stacks = [lm.transformer] if hasattr(lm, "transformer") else \
        [s for s in (getattr(lm, "encoder", None), getattr(lm, "decoder", None)) if s is not None]
    return [layer.mlp.gate for stack in stacks for layer in stack.layers]


def add_balance_log(model, writer, iteration):
    r"""Write the rank-averaged balance losses of all layers (no pipeline parallelism: every
    rank must hold every layer)."""
    from megatron import is_last_rank
    collected = [g.get_loss(clear=True).detach().reshape(-1) for g in _moe_gates(model) if g.has_loss]
    if not collected:
        return
    per_metric = torch.stack(collected, dim=1)              # [metrics, layers]
    group = get_torch_default_comm()
    dist.all_reduce(per_metric, group=group)
    per_metric /= dist.get_world_size(group=group)
    if not (writer and is_last_rank()):
        return
    names = list(balance_dict) or ["loss"]
    for name, values in zip(names, per_metric):
        for layer_id, value in enumerate(values.tolist()):
            writer.add_scalar("balance-%s/layer-%d" % (name, layer_id), value, iteration)
        writer.add_scalar("balance-%s/all" % name, float(values.mean()), iteration)
