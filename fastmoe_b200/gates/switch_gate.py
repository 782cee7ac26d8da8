r"""
Top-1 routing with multiplicative-free logit jitter and a per-expert capacity, after the Switch
Transformer (Fedus et al., 2021).

Parity: ``fmoe/gates/switch_gate.py:12-59`` — same constructor (``topk`` must be 1,
``switch_eps``, ``capacity=(train rate, eval rate)``), same score definition (softmax over ALL
experts in fp32, the winner's probability is the score), same capacity rule
(``ceil(rate * B / num_expert)`` tokens per local expert, enforced across ranks, overflow
dropped with id -1) and the same balance loss
(``tot_expert * sum_e fraction_e * mean_prob_e`` over the kept tokens).
"""
import math

import torch

from .naive_gate import NaiveGate
from .utils import limit_by_capacity


class SwitchGate(NaiveGate):

    def __init__(self, d_model, num_expert, world_size, topk=1, switch_eps=.1,
                 capacity=(1.2, 2.4), gate_bias=True):
        if topk != 1:
            raise AssertionError("topk should be 1 in switch")
        super().__init__(d_model, num_expert, world_size, top_k=1, gate_bias=gate_bias)
        self.switch_eps, self.capacity = switch_eps, capacity

    def _jitter(self, logits):
        r"""Training only: add ``U(1 - eps, 1 + eps)`` to every logit."""
        if not self.training:
            return logits
        eps = self.switch_eps
        return logits + torch.empty_like(logits).uniform_(1.0 - eps, 1.0 + eps)

    def _slots_per_expert(self, n_tokens):
        rate = self.capacity[0] if self.training else self.capacity[1]
        return math.ceil(rate * n_tokens / self.num_expert)

    def _balance_loss(self, prob, winner):
        r"""Without boolean indexing (no device-to-host read, so the gate can sit in a CUDA graph)."""
        ids = winner.reshape(-1)
        kept = (ids >= 0).to(prob.dtype)
        n_kept = kept.sum().clamp(min=1.0)
        share = torch.zeros(self.tot_expert, dtype=prob.dtype, device=prob.device)
        share.scatter_add_(0, ids.clamp(min=0), kept)
        return self.tot_expert * ((share / n_kept) * (prob.sum(dim=0) / n_kept)).sum()

    def forward(self, inp):
        prob = torch.softmax(self._jitter(self.gate(inp)).float(), dim=-1)
        score, winner = prob.max(dim=-1, keepdim=True)
        _, _, winner = limit_by_capacity(winner, self.num_expert, self.world_size,
                                         self._slots_per_expert(inp.shape[0]),
                                         group=getattr(self, "moe_group", None))
        self.set_loss(self._balance_loss(prob, winner))
        return winner, score.to(inp.dtype)
