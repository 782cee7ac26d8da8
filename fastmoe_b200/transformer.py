r"""
MoE replacement of a Transformer feed-forward block.

Parity: ``fmoe/transformer.py`` — ``_Expert`` (``:11-31``) and ``FMoETransformerMLP``
(``:34-66``).  The reference builds ``num_expert`` separate one-expert modules
(``:51-55``), so every local expert runs alone between host synchronisations.  Here the
experts are one fused module whose parameters have the layout

    experts.htoh4.weight [E, d_hidden, d_model]   experts.htoh4.bias [E, d_hidden]
    experts.h4toh.weight [E, d_model, d_hidden]   experts.h4toh.bias [E, d_model]

and checkpoints written by the reference's per-expert layout
(``experts.{i}.htoh4.weight [1, d_hidden, d_model]`` …) are accepted on load.  On a B200
with bf16/fp16 data the whole layer — dispatch, both expert GEMMs with the activation,
combine — runs in the fused kernels of :mod:`fastmoe_b200.ops.fused`.
"""
import re

import torch
import torch.nn as nn

from .layers import FMoE
from .linear import FMoELinear

_PER_EXPERT_KEY = re.compile(r"^(.*experts\.)(\d+)\.(htoh4|h4toh)\.(weight|bias)$")


def activation_kind(act):
    r"""Name of an activation the fused GEMM epilogue implements, or ``None``."""
    if isinstance(act, nn.GELU):
        return "gelu_tanh" if getattr(act, "approximate", "none") == "tanh" else "gelu"
    if isinstance(act, nn.ReLU):
        return "relu"
    if isinstance(act, nn.Identity):
        return "identity"
    if act is torch.nn.functional.gelu:
        return "gelu"
    if act is torch.nn.functional.relu or act is torch.relu:
        return "relu"
    return None


class _Expert(nn.Module):
    r"""``num_expert`` two-layer MLPs: ``htoh4`` → activation → ``h4toh``."""

    def __init__(self, num_expert, d_model, d_hidden, activation, rank=0):
        super().__init__()
        self.htoh4 = FMoELinear(num_expert, d_model, d_hidden, bias=True, rank=rank)
        self.h4toh = FMoELinear(num_expert, d_hidden, d_model, bias=True, rank=rank)
        self.activation = activation

    def forward(self, inp, fwd_expert_count):
        x = self.htoh4(inp, fwd_expert_count)
        x = self.activation(x)
        return self.h4toh(x, fwd_expert_count)

    def forward_single(self, inp, fwd_expert_count, idx):
        r"""Expert ``idx`` alone on ``inp`` (all rows belong to it)."""
        w1, b1 = self.htoh4.weight[idx], self.htoh4.bias[idx]
        w2, b2 = self.h4toh.weight[idx], self.h4toh.bias[idx]
        x = torch.nn.functional.linear(inp.type_as(w1), w1, b1)
        x = self.activation(x)
        return torch.nn.functional.linear(x, w2, b2)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict,
                              missing_keys, unexpected_keys, error_msgs):
        # Checkpoints of the reference's ModuleList layout carry keys
        # `<prefix>{i}.htoh4.weight` of shape [1, out, in]; stack them into the fused layout.
        groups = {}
        for key in list(state_dict.keys()):
            if not key.startswith(prefix):
                continue
            m = _PER_EXPERT_KEY.match(key)
            if m is None or m.group(1) != prefix:
                continue
            groups.setdefault((m.group(3), m.group(4)), {})[int(m.group(2))] = state_dict.pop(key)
        for (layer, kind), parts in groups.items():
            stacked = torch.cat([parts[i] for i in sorted(parts)], dim=0)
            state_dict[prefix + layer + "." + kind] = stacked
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict,
                                      missing_keys, unexpected_keys, error_msgs)


def per_expert_state_dict(state_dict):
    r"""Rewrite fused expert keys into the reference's per-expert ModuleList layout.

    ``…experts.htoh4.weight [E,h,d]`` becomes ``…experts.{i}.htoh4.weight [1,h,d]`` for
    ``i < E``; other entries are passed through.  Use it to hand a checkpoint to code that
    expects what ``fmoe/transformer.py:51-55`` produces.
    """
    out = type(state_dict)()
    pat = re.compile(r"^(.*experts\.)(htoh4|h4toh)\.(weight|bias)$")
    for key, value in state_dict.items():
        m = pat.match(key)
        if m is None:
            out[key] = value
            continue
        for i in range(value.shape[0]):
            out["%s%d.%s.%s" % (m.group(1), i, m.group(2), m.group(3))] = value[i:i + 1]
    return out


class FMoETransformerMLP(FMoE):
    r"""A complete MoE MLP block: ``[..., d_model] → [..., d_model]``.

    * ``activation``: module applied between the two expert linears.  GELU (erf or tanh),
      ReLU and Identity are fused into the first GEMM's epilogue on the GPU; anything else
      (e.g. ``Sequential(ReLU, Dropout)``) runs as a PyTorch op between two grouped GEMMs.
    * ``d_hidden``: hidden size of each expert.
    * ``expert_dp_comm``: gradient-reduction group name of the expert parameters.
    * ``expert_rank``: accepted and ignored, as in the reference.
    """

    def __init__(self, num_expert=32, d_model=1024, d_hidden=4096, activation=torch.nn.GELU(),
                 expert_dp_comm="none", expert_rank=0, **kwargs):
        super().__init__(num_expert=num_expert, d_model=d_model, expert=None, **kwargs)
        self.d_hidden = d_hidden
        self.experts = _Expert(self.num_expert, d_model, d_hidden, activation, rank=expert_rank)
        self.mark_parallel_comm(expert_dp_comm)

    def _fused_forward(self, moe_inp, gate_top_k_idx, gate_score):
        if not torch.is_tensor(moe_inp) or not moe_inp.is_cuda:
            return None
        from . import config
        from .ops import fused
        if not fused.supports(self, moe_inp, gate_top_k_idx):
            return None
        if (config.faster_schedule_enabled() and config.faster_shadow_enabled()
                and self.world_size > 1):
            # shadow experts stay on the fused path: masked out of the exchange, computed
            # locally with broadcast parameters
            from .fastermoe import fused_shadow
            return fused_shadow.moe_mlp_forward(self, moe_inp, gate_top_k_idx, gate_score)
        return fused.moe_mlp_forward(self, moe_inp, gate_top_k_idx, gate_score)

    def forward(self, inp: torch.Tensor):
        original_shape = inp.shape
        out = super().forward(inp.reshape(-1, self.d_model))
        return out.reshape(original_shape)
