r"""GShard top-2 gate with local capacity and random second-expert routing.

Parity: ``fmoe/gates/gshard_gate.py:12-49``.
"""
import math

import torch
import torch.nn.functional as F

from .naive_gate import NaiveGate
from ..ops import api as _ops


def gshard_balance_loss(logits, top1_idx, tot_expert, num_expert):
    r"""``mean(c_e · m_e) · num_expert²`` with ``c_e`` the fraction of tokens whose first choice
    is expert ``e`` and ``m_e`` the mean softmax probability of ``e``."""
    n = logits.shape[0]
    # scatter_add instead of bincount: no device->host read, so the gate can be graph-captured
    c_e = torch.zeros(tot_expert, device=logits.device).scatter_add_(
        0, top1_idx, torch.ones_like(top1_idx, dtype=torch.float32)) / n
    m_e = F.softmax(logits, dim=1).mean(dim=0)
    return torch.mean(c_e * m_e.float()) * (num_expert ** 2)


def drop_second_expert_randomly(topk_idx, topk_val):
    r"""GShard random routing: the 2nd expert is kept with probability ``2 · score₂``."""
    u = torch.rand(topk_val.shape[0], device=topk_val.device)
    topk_idx[:, 1].masked_fill_(2 * topk_val[:, 1] < u, -1)
    return topk_idx


class GShardGate(NaiveGate):
    r"""Top-2 gate; per-global-expert capacity ``ceil(rate·B)·2 // tot_expert`` applied to this
    rank's own tokens; ``rate = capacity[0]`` in training, ``capacity[1]`` in eval."""

    def __init__(self, d_model, num_expert, world_size, topk=2, capacity=(1.2, 2.4),
                 random_routing=True, gate_bias=True):
        assert topk == 2, "topk should be 2 in gshard"
        super().__init__(d_model, num_expert, world_size, top_k=2, gate_bias=gate_bias)
        self.capacity = capacity
        self.random_routing = random_routing

    def forward(self, x):
        topk_idx, topk_val, logits = super().forward(x, return_all_scores=True)
        logits = logits.view(-1, self.tot_expert)
        self.set_loss(gshard_balance_loss(logits, topk_idx[:, 0], self.tot_expert, self.num_expert))

        rate = self.capacity[0 if self.training else 1]
        cap = math.ceil(rate * x.shape[0]) * self.top_k // self.tot_expert
        cap_t = torch.full((self.tot_expert,), cap, dtype=torch.int32, device=topk_idx.device)
        topk_idx = _ops.prune_gate_by_capacity(topk_idx, cap_t, self.num_expert, self.world_size)

        if self.random_routing:
            topk_idx = drop_second_expert_randomly(topk_idx, topk_val)
        return topk_idx, topk_val
