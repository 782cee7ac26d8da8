r"""Degenerate gate: every slot goes to global expert 0 (parity: ``fmoe/gates/zero_gate.py:11-30``)."""
import torch

from .base_gate import BaseGate


class ZeroGate(BaseGate):
    r"""Routes all ``top_k`` slots of every token to expert 0 with weight ``1/top_k``.

    The ids are returned flattened (``[B·k]``) like the reference does; ``FMoE`` restores
    the ``[B, k]`` view.
    """

    def __init__(self, _1, num_expert, world_size, top_k=2):
        super().__init__(num_expert, world_size)
        self.top_k = top_k

    def forward(self, inp):
        n = inp.shape[0]
        idx = inp.new_zeros(n * self.top_k, dtype=torch.int64)
        score = torch.full((n, 1, self.top_k), 1.0 / self.top_k, device=inp.device)
        return idx, score
