r"""
Routing policies ("gates").

Every gate maps ``x [B, d_model]`` to ``(topk_idx int64 [B, k], topk_score [B, k])`` where
``topk_idx`` holds **global** expert ids (``rank * num_expert + local id``) and ``-1`` marks
a dropped slot; a balance loss, if any, is left in ``gate.get_loss()``.
Exported names match ``fmoe/gates/__init__.py:4-12``; ``FasterGate`` additionally lives in
:mod:`fastmoe_b200.gates.faster_gate` as in the reference.
"""
from .base_gate import BaseGate
from .zero_gate import ZeroGate
from .naive_gate import NaiveGate
from .noisy_gate import NoisyGate
from .gshard_gate import GShardGate
from .switch_gate import SwitchGate
from .dc_gate import DCGate
from .swipe_gate import SwipeGate
from .faster_gate import FasterGate, gen_faster_gate

__all__ = ["BaseGate", "ZeroGate", "NaiveGate", "NoisyGate", "GShardGate", "SwitchGate",
           "DCGate", "SwipeGate", "FasterGate", "gen_faster_gate"]
