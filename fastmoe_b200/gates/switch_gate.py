r"""Switch-Transformer top-1 gate (parity: ``fmoe/gates/switch_gate.py:12-59``)."""
import math

import torch
import torch.nn.functional as F

from .naive_gate import NaiveGate
from .utils import limit_by_capacity


class SwitchGate(NaiveGate):
    r"""Top-1 routing on an fp32 softmax over all experts.

    Training adds noise drawn from ``U(1-eps, 1+eps)`` to the logits.  Each local expert
    accepts ``ceil(rate · B / num_expert)`` tokens over all ranks.  Loss:
    ``Σ_e fraction_e · prob_e · tot_expert`` over the kept tokens.
    """

    def __init__(self, d_model, num_expert, world_size, topk=1, switch_eps=.1,
                 capacity=(1.2, 2.4), gate_bias=True):
        assert topk == 1, "topk should be 1 in switch"
        super().__init__(d_model, num_expert, world_size, top_k=1, gate_bias=gate_bias)
        self.switch_eps = switch_eps
        self.capacity = capacity

    def forward(self, inp):
        logits = self.gate(inp)
        if self.training:
            noise = torch.rand_like(logits) * (2 * self.switch_eps) + (1.0 - self.switch_eps)
            logits = logits + noise
        prob = F.softmax(logits.float(), dim=-1)
        top1_score, top1_idx = torch.topk(prob, k=1, dim=-1, largest=True)
        top1_score = top1_score.to(dtype=inp.dtype)

        rate = self.capacity[0 if self.training else 1]
        cap = math.ceil(rate * inp.shape[0] / self.num_expert)
        _lec, _gec, top1_idx = limit_by_capacity(top1_idx, self.num_expert, self.world_size, cap)

        # mask arithmetic instead of boolean indexing: no device->host read
        flat = top1_idx.reshape(-1)
        kept = (flat > -1).float()
        n_kept = kept.sum().clamp(min=1.0)
        fraction = torch.zeros(self.tot_expert, device=inp.device).scatter_add_(
            0, flat.clamp(min=0), kept) / n_kept
        prob_expert = prob.sum(dim=0) / n_kept
        self.set_loss((fraction * prob_expert).sum() * self.tot_expert)
        return top1_idx, top1_score
