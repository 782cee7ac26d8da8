r"""
MoE layers shaped for Megatron-LM (parity: ``fmoe/megatron/layers.py``).

``MegatronMLP`` (``:71-155`` there) is an ``FMoETransformerMLP`` whose expert-parallel group is
Megatron's data-parallel group, whose gate follows ``--balance-strategy`` and whose forward
returns ``(output, bias)`` like Megatron's ``ParallelMLP``.  ``fmoefy`` (``:158-224``) installs
it in every transformer layer of a v2.2 / v2.5 / v3.0.2 model.
"""
import math

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from ..transformer import FMoETransformerMLP
from .balance import generate_megatron_gate_hook, reset_gate_hook


class _FakeMegatronMLP(nn.Module):
    r"""Dense two-layer MLP with Megatron's ``(output, bias)`` return, for correctness tests."""

    def __init__(self, args, _):
        super().__init__()
        self.fc1 = nn.Linear(args.hidden_size, args.hidden_hidden_size)
        self.fc2 = nn.Linear(args.hidden_hidden_size, args.hidden_size)

    def forward(self, x):
        x = self.fc2(F.gelu(self.fc1(x)))
        return x, torch.zeros_like(x)


def _megatron_init_method(self, rng, sigma):
    r"""``weight ~ N(0, sigma)`` from a numpy generator, zero bias (Megatron's init)."""
    w = rng.normal(loc=0.0, scale=sigma, size=tuple(self.weight.size()))
    self.weight.data = torch.from_numpy(w).to(dtype=self.weight.dtype, device=self.weight.device)
    if self.bias is not None:
        with torch.no_grad():
            self.bias.zero_()


def _random_init_weight(self, rng):
    r"""kaiming-uniform(a=√5) weight and uniform bias drawn from a numpy generator."""
    fan_in = self.weight[0].shape[-1]
    gain = nn.init.calculate_gain("leaky_relu", math.sqrt(5))
    bound = math.sqrt(3.0) * gain / math.sqrt(fan_in)
    w = rng.uniform(-bound, bound, size=tuple(self.weight.size()))
    self.weight.data = torch.from_numpy(w).to(dtype=self.weight.dtype, device=self.weight.device)
    if self.bias is not None:
        b_bound = 1 / math.sqrt(fan_in)
        b = rng.uniform(-b_bound, b_bound, size=tuple(self.bias.size()))
        self.bias.data = torch.from_numpy(b).to(dtype=self.bias.dtype, device=self.bias.device)


_GATES = {"naive": "NaiveGate", "noisy": "NoisyGate", "gshard": "GShardGate",
          "switch": "SwitchGate", "swipe": "SwipeGate"}


class MegatronMLP(FMoETransformerMLP):
    r"""Drop-in for ``layer.mlp``: experts spread over Megatron's data-parallel group."""

    def __init__(self, args, layer_idx, gate=None):
        from .. import gates as gate_lib
        if not args.distributed_experts:
            world_size, moe_group = 1, None
        else:
            from megatron.mpu import get_data_parallel_group
            world_size, moe_group = args.data_parallel_size, get_data_parallel_group()

        strategy = args.balance_strategy or "naive"
        if strategy in _GATES:
            gate = getattr(gate_lib, _GATES[strategy])
        elif gate is None:
            raise AssertionError("Undefined balance strategy %s" % strategy)

        super().__init__(
            args.fmoe_num_experts,
            top_k=args.top_k,
            d_model=args.hidden_size,
            d_hidden=args.hidden_hidden_size,
            world_size=world_size,
            moe_group=moe_group,
            expert_dp_comm="none" if args.distributed_experts else "dp",
            gate_hook=generate_megatron_gate_hook(layer_idx, args.fmoe_num_experts * world_size),
            gate=gate,
        )
        self.hidden_size = args.hidden_size
        self.rank = args.rank if args.distributed_experts else 0
        self.sigma = args.init_method_std
        self.num_layers = args.num_layers
        self.reset_parameters()

    def reset_parameters(self):
        r"""Megatron seeds torch identically on all ranks, so a numpy generator offset by the
        rank gives every rank different experts."""
        rng = np.random.default_rng(np.random.randint(2048) + self.rank)
        experts = list(self.experts) if isinstance(self.experts, nn.ModuleList) else [self.experts]
        for e in experts:
            _megatron_init_method(e.htoh4, rng, self.sigma)
        out_std = self.sigma / math.sqrt(2.0 * self.num_layers)
        for e in experts:
            _megatron_init_method(e.h4toh, rng, out_std)

    def forward(self, inp):
        from megatron import mpu
        out = mpu.reduce_from_tensor_model_parallel_region(super().forward(inp))
        return out, torch.zeros(self.hidden_size, dtype=inp.dtype, device=inp.device)


def fmoefy(model, fmoe_num_experts=None, distributed_experts=True, hidden_hidden_size=None,
           top_k=None, gate=None, megatron_version=None):
    r"""Replace ``layer.mlp`` of every transformer layer of a Megatron model by ``MegatronMLP``.

    ``megatron_version`` selects where the layers live: ``"v2.2"`` →
    ``model.language_model.transformer.layers``; ``"v2.5"`` / ``"v3.0.2"`` →
    ``model.language_model.encoder.layers`` (and ``decoder.layers`` when present).
    With ``distributed_experts=False`` all ranks hold the same experts (plain data parallel).
    """
    from megatron import get_args
    args = get_args()
    if distributed_experts is not None:
        args.distributed_experts = distributed_experts
    if fmoe_num_experts is not None:
        args.fmoe_num_experts = fmoe_num_experts
    assert getattr(args, "fmoe_num_experts", None) is not None, \
        "fmoe_num_experts should be specified in arguments or fmoefy function"
    if top_k is not None:
        args.top_k = top_k
    elif not hasattr(args, "top_k"):
        args.top_k = 2
    args.hidden_hidden_size = hidden_hidden_size

    lm = model.language_model
    if megatron_version == "v2.2":
        stacks = [lm.transformer.layers]
    elif megatron_version in ("v2.5", "v3.0.2"):
        stacks = [lm.encoder.layers]
        if getattr(lm, "decoder", None) is not None:
            stacks.append(lm.decoder.layers)
    else:
        raise AssertionError(f"megatron_version {megatron_version} not known.")
    num_layers = 0
    for stack in stacks:
        for idx, layer in enumerate(stack):
            layer.mlp = MegatronMLP(args, idx, gate=gate)
        num_layers += len(stack)
    reset_gate_hook(num_layers)
    return model
