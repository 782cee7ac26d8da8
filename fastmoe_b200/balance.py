r"""
Load-balance metrics.

Parity: ``fmoe/balance.py`` — the ``metrics`` dictionary (``:4-8``) and
``reset_balance_profile`` (``:11-15``).  ``update_balance_profile`` is an empty stub in the
reference (``:18-28``); here it records the metrics from the per-expert token counts.
"""
import torch

metrics = {
    "coefficient-variation": lambda c_e: torch.std(c_e) / torch.mean(c_e),
    "Lmax-over-Lmin": lambda c_e: (torch.max(c_e) + 1) / (torch.min(c_e) + 1),
    "Lmax-over-Lmean": lambda c_e: torch.max(c_e) / torch.mean(c_e),
}


def reset_balance_profile(balance_dict, num_layers, balance_strategy):
    for key in metrics:
        balance_dict[key] = [None for _ in range(num_layers)]
    if balance_strategy:
        balance_dict[f"{balance_strategy}_loss"] = [None for _ in range(num_layers)]


def update_balance_profile(balance_dict, gate_top_k_idx, _gate_score_top_k, gate_context,
                           layer_idx, num_expert, balance_strategy):
    r"""Store the balance metrics of one layer call; ``gate_context`` may carry the gate loss."""
    with torch.no_grad():
        idx = gate_top_k_idx.reshape(-1)
        idx = idx[idx >= 0]
        c_e = torch.bincount(idx, minlength=num_expert)[:num_expert].float()
        for key, fn in metrics.items():
            if key in balance_dict:
                balance_dict[key][layer_idx] = fn(c_e)
        loss_key = f"{balance_strategy}_loss" if balance_strategy else None
        if loss_key and loss_key in balance_dict and gate_context is not None:
            balance_dict[loss_key][layer_idx] = gate_context
