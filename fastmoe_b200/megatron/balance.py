r"""Balance-loss monitoring inside Megatron (parity: ``fmoe/megatron/balance.py:11-78``)."""
import torch

from ..balance import reset_balance_profile, update_balance_profile
from ..parallel.comm import get_torch_default_comm

balance_dict = {}
num_layers = 0


def _args():
    from megatron import get_args
    return get_args()


def reset_gate_hook(_num_layers=None):
    global num_layers
    if _num_layers is not None:
        num_layers = _num_layers
    reset_balance_profile(balance_dict, num_layers, _args().balance_strategy)


def get_balance_profile():
    return balance_dict


def generate_megatron_gate_hook(layer_idx, num_expert_global):
    r"""Gate hook that records the balance metrics of layer ``layer_idx`` on every call."""
    strategy = _args().balance_strategy

    def megatron_gate_hook(gate_top_k_idx, gate_score_top_k, gate_context):
        update_balance_profile(balance_dict, gate_top_k_idx, gate_score_top_k, gate_context,
                               layer_idx, num_expert_global, strategy)

    return megatron_gate_hook


def _transformer_layers(model):
    lm = model.language_model
    if hasattr(lm, "transformer"):
        return list(lm.transformer.layers)
    layers = list(lm.encoder.layers)
    if getattr(lm, "decoder", None) is not None:
        layers += list(lm.decoder.layers)
    return layers


def add_balance_log(model, writer, iteration):
    r"""All-reduce the layers' balance losses and write them as TensorBoard scalars
    ``balance-{metric}/layer-{i}`` and ``balance-{metric}/all`` (no pipeline parallelism)."""
    from megatron import is_last_rank
    while hasattr(model, "module"):
        model = model.module
    losses = [l.mlp.gate.get_loss(clear=True) for l in _transformer_layers(model) if l.mlp.gate.has_loss]
    if not losses:
        return
    table = torch.vstack([x.reshape(1, -1) for x in losses]).detach().t().contiguous()
    group = get_torch_default_comm()
    torch.distributed.all_reduce(table, group=group)
    table /= torch.distributed.get_world_size(group=group)
    if writer and is_last_rank():
        names = list(balance_dict.keys()) or ["loss"]
        for row, name in zip(table, names):
            for layer_id, val in enumerate(row):
                writer.add_scalar(f"balance-{name}/layer-{layer_id}", val.item(), iteration)
            writer.add_scalar(f"balance-{name}/all", row.mean().item(), iteration)
