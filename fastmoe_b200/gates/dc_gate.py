r"""Distributed-capacity gate: GShard loss, capacity enforced on the *global* load of each expert.

Parity: ``fmoe/gates/dc_gate.py:14-48``.
"""
import math

from .gshard_gate import drop_second_expert_randomly, gshard_balance_loss
from .naive_gate import NaiveGate
from .utils import limit_by_capacity


class DCGate(NaiveGate):
    r"""Top-2 gate; every expert accepts at most ``ceil(rate·B)`` tokens summed over all ranks."""

    def __init__(self, d_model, num_expert, world_size, topk=2, capacity=(1.2, 2.4),
                 random_routing=True, gate_bias=True):
        assert topk == 2, "topk should be 2 in DCGate"
        super().__init__(d_model, num_expert, world_size, top_k=2, gate_bias=gate_bias)
        self.capacity = capacity
        self.random_routing = random_routing

    def forward(self, x):
        topk_idx, topk_val, logits = super().forward(x, return_all_scores=True)
        logits = logits.view(-1, self.tot_expert)
        self.set_loss(gshard_balance_loss(logits, topk_idx[:, 0], self.tot_expert, self.num_expert))

        rate = self.capacity[0 if self.training else 1]
        cap = math.ceil(rate * x.shape[0])
        _lec, _gec, topk_idx = limit_by_capacity(topk_idx, self.num_expert, self.world_size, cap)

        if self.random_routing:
            topk_idx = drop_second_expert_randomly(topk_idx, topk_val)
        return topk_idx, topk_val
