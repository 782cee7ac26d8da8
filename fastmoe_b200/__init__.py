r"""
fastmoe_b200 — a Mixture-of-Experts training system for NVIDIA B200 (sm_100a).

The public surface is that of FastMoE (``fmoe/__init__.py:5-8``): ``FMoE``,
``FMoELinear``, ``FMoETransformerMLP`` and ``DistributedGroupedDataParallel``; the package
can also be imported under the name ``fmoe``.
"""
from .layers import FMoE
from .linear import FMoELinear
from .transformer import FMoETransformerMLP
from .distributed import DistributedGroupedDataParallel

__version__ = "0.2.0"
__all__ = ["FMoE", "FMoELinear", "FMoETransformerMLP", "DistributedGroupedDataParallel"]
