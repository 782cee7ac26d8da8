r"""
SWIPE: a top-k gate whose training-time routing never overloads a worker.

Parity: ``fmoe/gates/swipe_gate.py:15-49``.  Every worker can take ``B * top_k`` tokens per
step.  The k choices of a token are balanced one rank of choice after the other: all first
choices are offered to their workers, which accept them in rank order until full; the rejected
tokens are "swiped" to workers that still have room (to their expert ``j % num_expert`` for the
j-th choice); then the second choices go through the same procedure with the capacity that is
left, and so on.  Scores are the softmax over the logits of the experts finally chosen.
Evaluation keeps the plain top-k.  The expert-parallel group must exist (``ensure_comm``)
before the first training call.
"""
import torch

from .naive_gate import NaiveGate
from ..ops import api as _ops
from ..ops import gating


class SwipeGate(NaiveGate):

    def __init__(self, d_model, num_expert, world_size, top_k=2, gate_bias=True):
        super().__init__(d_model, num_expert, world_size, top_k=top_k, gate_bias=gate_bias)

    def swipe_once(self, idx, capacity, bias):
        r"""Balance one choice of every token; returns the new expert ids and what capacity is left."""
        with torch.no_grad():
            moved, left = _ops.swipe_once(idx, capacity, self.num_expert, self.world_size, bias)
        return moved.to(idx.device), left

    def _balanced_choices(self, preferred):
        r"""``preferred [B, k]`` (descending preference) → balanced ids ``[B, k]``."""
        left = torch.full((1,), preferred.shape[0] * self.top_k, dtype=torch.long, device=preferred.device)
        columns = []
        for choice in range(self.top_k):
            ids, left = self.swipe_once(preferred[:, choice], left, choice % self.num_expert)
            columns.append(ids)
        return torch.stack(columns, dim=1)

    def forward(self, inp):
        logits = self.gate(inp)
        if not self.training:
            return gating.topk_softmax(logits, self.top_k)
        preferred = torch.topk(logits, k=self.top_k, dim=-1).indices
        chosen = self._balanced_choices(preferred)
        scores = torch.softmax(torch.gather(logits, 1, chosen), dim=-1)
        return chosen, scores
