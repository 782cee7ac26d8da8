r"""SWIPE-balanced gate (parity: ``fmoe/gates/swipe_gate.py:15-49``)."""
import torch
import torch.nn.functional as F

from .naive_gate import NaiveGate
from ..ops import api as _ops


class SwipeGate(NaiveGate):
    r"""Top-k gate whose training-time routing is re-balanced so that no worker receives more
    than ``B·top_k`` tokens: overflow is swiped to expert ``j % num_expert`` of workers with room.
    Evaluation is a plain top-k.  Needs the expert-parallel group (``ensure_comm``) first.
    """

    def __init__(self, d_model, num_expert, world_size, top_k=2, gate_bias=True):
        super().__init__(d_model, num_expert, world_size, top_k, gate_bias)

    def swipe_once(self, idx, capacity, bias):
        with torch.no_grad():
            new_idx, capacity = _ops.swipe_once(idx, capacity, self.num_expert, self.world_size, bias)
        return new_idx.to(idx.device), capacity

    def forward(self, inp):
        logits = self.gate(inp)
        top_val, top_idx = torch.topk(logits, k=self.top_k, dim=-1)
        if not self.training:
            return top_idx, F.softmax(top_val, dim=-1)

        capacity = torch.scalar_tensor(inp.shape[0] * self.top_k, dtype=torch.long)
        rows = torch.arange(inp.shape[0], device=inp.device)
        new_idx, new_val = [], []
        for j in range(self.top_k):
            idx_j, capacity = self.swipe_once(top_idx[:, j], capacity, j % self.num_expert)
            new_idx.append(idx_j)
            new_val.append(logits[rows, idx_j])
        topk_idx = torch.stack(new_idx, dim=1)
        topk_val = F.softmax(torch.stack(new_val, dim=1), dim=-1)
        return topk_idx, topk_val
