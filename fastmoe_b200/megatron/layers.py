r"""
MoE layers shaped for Megatron-LM.

Parity: ``fmoe/megatron/layers.py``.  :class:`MegatronMLP` (``:71-155`` there) is an
``FMoETransformerMLP`` whose expert-parallel group is Megatron's data-parallel group, whose gate
follows ``--balance-strategy``, whose experts are initialised the way Megatron initialises its
MLP (``N(0, sigma)`` for the first linear, ``N(0, sigma / sqrt(2 L))`` for the second, zero
biases, different experts on different ranks) and whose ``forward`` returns ``(output, bias)``
like Megatron's ``ParallelMLP``, after summing the tensor-parallel partial outputs.
:func:`fmoefy` (``:158-224``) installs it in every transformer layer of a v2.2 / v2.5 / v3.0.2
model.  :class:`_FakeMegatronMLP` is the dense stand-in the reference keeps for correctness
tests.
"""
import math

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from ..transformer import FMoETransformerMLP
from .balance import generate_megatron_gate_hook, reset_gate_hook

# --balance-strategy value -> gate class of fastmoe_b200.gates
_GATES = {"naive": "NaiveGate", "noisy": "NoisyGate", "gshard": "GShardGate",
          "switch": "SwitchGate", "swipe": "SwipeGate"}
# Megatron release -> attribute path(s) of the transformer layer lists below `language_model`
_LAYER_STACKS = {"v2.2": ("transformer",), "v2.5": ("encoder", "decoder"), "v3.0.2": ("encoder", "decoder")}


class _FakeMegatronMLP(nn.Module):
    r"""Dense two-layer GELU MLP with Megatron's ``(output, bias)`` return value."""

    def __init__(self, args, _layer_idx):
        super().__init__()
        self.fc1 = nn.Linear(args.hidden_size, args.hidden_hidden_size)
        self.fc2 = nn.Linear(args.hidden_hidden_size, args.hidden_size)

    def forward(self, x):
        y = self.fc2(F.gelu(self.fc1(x)))
        return y, torch.zeros_like(y)


def _assign_from_numpy(param, array):
    param.data = torch.from_numpy(array).to(dtype=param.dtype, device=param.device)


def _megatron_init_method(linear, rng, sigma):
    r"""Megatron's initialisation of a linear layer: ``weight ~ N(0, sigma)`` drawn from the numpy
    generator ``rng`` (so that ranks seeded alike in torch still get different experts), zero bias."""
    _assign_from_numpy(linear.weight, rng.normal(loc=0.0, scale=sigma, size=tuple(linear.weight.shape)))
    if linear.bias is not None:
        with torch.no_grad():
            linear.bias.zero_()


def _random_init_weight(linear, rng):
    r"""``nn.Linear``'s default initialisation (Kaiming-uniform with ``a = sqrt 5``, uniform bias)
    drawn from a numpy generator; the fan-in is that of one expert's ``[out, in]`` matrix."""
    fan_in = linear.weight.shape[-1]
    w_bound = math.sqrt(3.0) * nn.init.calculate_gain("leaky_relu", math.sqrt(5)) / math.sqrt(fan_in)
    _assign_from_numpy(linear.weight, rng.uniform(-w_bound, w_bound, size=tuple(linear.weight.shape)))
    if linear.bias is not None:
        b_bound = 1.0 / math.sqrt(fan_in)
        _assign_from_numpy(linear.bias, rng.uniform(-b_bound, b_bound, size=tuple(linear.bias.shape)))


def _expert_modules(experts):
    return list(experts) if isinstance(experts, nn.ModuleList) else [experts]


class MegatronMLP(FMoETransformerMLP):
    r"""Drop-in for ``layer.mlp``: experts spread over (or replicated in) Megatron's data-parallel
    group, gate chosen by ``args.balance_strategy``."""

    def __init__(self, args, layer_idx, gate=None):
        from .. import gates as gate_lib
        spread = bool(args.distributed_experts)
        if spread:
            from megatron.mpu import get_data_parallel_group
            world_size, moe_group = args.data_parallel_size, get_data_parallel_group()
        else:
            world_size, moe_group = 1, None

        strategy = args.balance_strategy or "naive"
        if strategy in _GATES:
            gate = getattr(gate_lib, _GATES[strategy])
        elif gate is None:
            raise AssertionError("Undefined balance strategy %s" % strategy)

        super().__init__(
            args.fmoe_num_experts, d_model=args.hidden_size, d_hidden=args.hidden_hidden_size,
            top_k=args.top_k, world_size=world_size, moe_group=moe_group,
            expert_dp_comm="none" if spread else "dp", gate=gate,
            gate_hook=generate_megatron_gate_hook(layer_idx, args.fmoe_num_experts * world_size))
        self.hidden_size = args.hidden_size
        self.rank = args.rank if spread else 0
        self.sigma = args.init_method_std
        self.num_layers = args.num_layers
        self.reset_parameters()

    def reset_parameters(self):
        r"""Megatron seeds torch identically on all ranks; offsetting a numpy generator by the rank
        gives every rank different experts (and replicas identical ones)."""
        rng = np.random.default_rng(np.random.randint(2048) + self.rank)
        modules = _expert_modules(self.experts)
        for m in modules:
            _megatron_init_method(m.htoh4, rng, self.sigma)
        scaled = self.sigma / math.sqrt(2.0 * self.num_layers)
        for m in modules:
            _megatron_init_method(m.h4toh, rng, scaled)

    def forward(self, inp):
        from megatron import mpu
        partial = super().forward(inp)
        out = mpu.reduce_from_tensor_model_parallel_region(partial)
        return out, torch.zeros(self.hidden_size, dtype=inp.dtype, device=inp.device)


def _layer_stacks(model, megatron_version):
    if megatron_version not in _LAYER_STACKS:
        raise AssertionError(f"megatron_version {megatron_version} not known.")
    lm = model.language_model
    stacks = [getattr(lm, name, None) for name in _LAYER_STACKS[megatron_version]]
    return [s.layers for s in stacks if s is not None]


def fmoefy(model, fmoe_num_experts=None, distributed_experts=True, hidden_hidden_size=None,
           top_k=None, gate=None, megatron_version=None):
    r"""Replace ``layer.mlp`` of every transformer layer of a Megatron model by :class:`MegatronMLP`.

    ``megatron_version``: ``"v2.2"`` (layers under ``language_model.transformer``) or ``"v2.5"`` /
    ``"v3.0.2"`` (``language_model.encoder`` and, when present, ``.decoder``).  Arguments that are
    given override the corresponding Megatron arguments; ``fmoe_num_experts`` must come from one
    of the two.  With ``distributed_experts=False`` all ranks hold the same experts (plain data
    parallelism).
    """
    from megatron import get_args
    args = get_args()
    for name, value in (("distributed_experts", distributed_experts),
                        ("fmoe_num_experts", fmoe_num_experts), ("top_k", top_k)):
        if value is not None:
            setattr(args, name, value)
    if getattr(args, "fmoe_num_experts", None) is None:
        raise AssertionError("fmoe_num_experts should be specified in arguments or fmoefy function")
    if not hasattr(args, "top_k"):
        args.top_k = 2
    args.hidden_hidden_size = hidden_hidden_size

    total = 0
    for layers in _layer_stacks(model, megatron_version):
        for idx, layer in enumerate(layers):
            layer.mlp = MegatronMLP(args, idx, gate=gate)
        total += len(layers)
    reset_gate_hook(total)
    return model
