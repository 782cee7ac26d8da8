r"""
A gate that sends everything to global expert 0.

Useful for tests (all other experts receive zero tokens) and as the simplest possible routing
policy.  Parity: ``fmoe/gates/zero_gate.py:11-30``: the first constructor argument (the model
width) is ignored, ids come back flattened as ``[B * top_k]`` and scores as ``[B, 1, top_k]``
with every slot weighted ``1 / top_k``; ``FMoE`` restores the ``[B, top_k]`` view of the ids.
"""
import torch

from .base_gate import BaseGate


class ZeroGate(BaseGate):

    def __init__(self, _d_model, num_expert, world_size, top_k=2):
        super().__init__(num_expert, world_size)
        self.top_k = top_k

    def forward(self, inp):
        n_slots = inp.shape[0] * self.top_k
        expert_ids = torch.zeros(n_slots, dtype=torch.int64, device=inp.device)
        weights = torch.full((inp.shape[0], 1, self.top_k), 1.0 / self.top_k, device=inp.device)
        return expert_ids, weights
