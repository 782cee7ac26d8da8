r"""
``import fmoe`` — the FastMoE import surface on top of :mod:`fastmoe_b200`.

Every submodule of the reference package (``fmoe.layers``, ``fmoe.linear``,
``fmoe.transformer``, ``fmoe.functions``, ``fmoe.distributed``, ``fmoe.utils``,
``fmoe.balance``, ``fmoe.gates.*``, ``fmoe.fastermoe.*``, ``fmoe.megatron.*``) resolves to the
module of the same name in ``fastmoe_b200``; user code written against FastMoE imports
unchanged.
"""
import importlib
import sys

import fastmoe_b200 as _impl
from fastmoe_b200 import (DistributedGroupedDataParallel, FMoE, FMoELinear,  # noqa: F401
                          FMoETransformerMLP)

_SUBMODULES = [
    "layers", "linear", "transformer", "functions", "distributed", "utils", "balance", "config",
    "checkpoint",
    "gates", "gates.base_gate", "gates.naive_gate", "gates.noisy_gate", "gates.gshard_gate",
    "gates.switch_gate", "gates.dc_gate", "gates.swipe_gate", "gates.zero_gate",
    "gates.faster_gate", "gates.utils",
    "fastermoe", "fastermoe.config", "fastermoe.expert_utils", "fastermoe.schedule",
    "fastermoe.shadow_policy",
]

for _name in _SUBMODULES:
    _mod = importlib.import_module("fastmoe_b200." + _name)
    sys.modules["fmoe." + _name] = _mod
    if "." not in _name:
        globals()[_name] = _mod


def __getattr__(name):
    # fmoe.megatron needs the `megatron` package (or its stand-in) only when it is used.
    if name == "megatron":
        mod = importlib.import_module("fastmoe_b200.megatron")
        sys.modules["fmoe.megatron"] = mod
        for sub in ("layers", "patch", "distributed", "checkpoint", "balance", "utils"):
            sys.modules["fmoe.megatron." + sub] = importlib.import_module("fastmoe_b200.megatron." + sub)
        return mod
    raise AttributeError(name)


__version__ = _impl.__version__
