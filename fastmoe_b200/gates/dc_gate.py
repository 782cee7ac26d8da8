r"""
Distributed-capacity gate.

GShard's top-2 policy and balance loss, but the capacity of an expert is a statement about its
*global* load: an expert accepts at most ``ceil(rate * B)`` tokens summed over all ranks
(``B`` = tokens of the calling rank), granted to the ranks in rank order, instead of a quota per
rank.  Parity: ``fmoe/gates/dc_gate.py:14-48`` (constructor, loss, capacity rule, optional
random dropping of weak second choices).
"""
import math

from . import gshard_gate as _gshard
from .naive_gate import NaiveGate
from .utils import limit_by_capacity


class DCGate(NaiveGate):

    def __init__(self, d_model, num_expert, world_size, topk=2, capacity=(1.2, 2.4),
                 random_routing=True, gate_bias=True):
        if topk != 2:
            raise AssertionError("topk should be 2 in DCGate")
        super().__init__(d_model, num_expert, world_size, top_k=2, gate_bias=gate_bias)
        self.capacity, self.random_routing = capacity, random_routing

    def global_capacity(self, n_tokens):
        r"""Tokens one expert may take from all ranks together."""
        rate = self.capacity[0] if self.training else self.capacity[1]
        return math.ceil(rate * n_tokens)

    def forward(self, x):
        experts, weights, logits = super().forward(x, return_all_scores=True)
        first_choice = experts[:, 0]
        self.set_loss(_gshard.gshard_balance_loss(logits.view(-1, self.tot_expert), first_choice,
                                                  self.tot_expert, self.num_expert))
        _, _, experts = limit_by_capacity(experts, self.num_expert, self.world_size,
                                          self.global_capacity(x.shape[0]),
                                          group=getattr(self, "moe_group", None))
        if self.random_routing:
            experts = _gshard.drop_second_expert_randomly(experts, weights)
        return experts, weights
