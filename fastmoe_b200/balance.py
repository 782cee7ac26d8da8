r"""
Load-balance metrics of a routing decision.

Parity: ``fmoe/balance.py`` — the ``metrics`` table (``:4-8``; same three names and formulas) and
``reset_balance_profile`` (``:11-15``).  The reference leaves ``update_balance_profile``
(``:18-28``) empty; here it computes the metrics from the per-expert token counts of a layer
call and stores them in the profile, which is a dictionary ``metric name -> [value per layer]``.
"""
import torch


def _coefficient_of_variation(load):
    return load.std() / load.mean()


def _max_over_min(load):
    # the +1 keeps the ratio finite for experts that received nothing
    return (load.max() + 1) / (load.min() + 1)


def _max_over_mean(load):
    return load.max() / load.mean()


# name -> function of the float vector ``load[e]`` (tokens routed to expert e)
metrics = {
    "coefficient-variation": _coefficient_of_variation,
    "Lmax-over-Lmin": _max_over_min,
    "Lmax-over-Lmean": _max_over_mean,
}


def _loss_key(balance_strategy):
    return "%s_loss" % balance_strategy if balance_strategy else None


def reset_balance_profile(balance_dict, num_layers, balance_strategy):
    r"""Fill ``balance_dict`` with one empty slot per layer for every metric (and for the gate's
    own balance loss when a strategy is named)."""
    names = list(metrics)
    if balance_strategy:
        names.append(_loss_key(balance_strategy))
    for name in names:
        balance_dict[name] = [None] * num_layers


def expert_load(gate_top_k_idx, num_expert):
    r"""Tokens per expert as a float vector; dropped slots (id -1) are not counted."""
    ids = gate_top_k_idx.reshape(-1)
    return torch.bincount(ids[ids >= 0], minlength=num_expert)[:num_expert].float()


def update_balance_profile(balance_dict, gate_top_k_idx, _gate_score_top_k, gate_context,
                           layer_idx, num_expert, balance_strategy):
    r"""Record the metrics of layer ``layer_idx``; ``gate_context``, when given, is stored as the
    layer's balance loss."""
    with torch.no_grad():
        load = expert_load(gate_top_k_idx, num_expert)
        for name, fn in metrics.items():
            if name in balance_dict:
                balance_dict[name][layer_idx] = fn(load)
    key = _loss_key(balance_strategy)
    if key is not None and key in balance_dict and gate_context is not None:
        balance_dict[key][layer_idx] = gate_context
