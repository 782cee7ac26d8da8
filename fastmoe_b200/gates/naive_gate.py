r"""Plain learned top-k gate (parity: ``fmoe/gates/naive_gate.py:11-45``)."""
import torch
import torch.nn as nn

from .base_gate import BaseGate
from ..ops import gating


class NaiveGate(BaseGate):
    r"""``Linear(d_model → tot_expert)``, top-k of the logits, softmax over the k selected logits.

    State-dict keys: ``gate.weight [tot_expert, d_model]``, ``gate.bias [tot_expert]``.
    On a GPU with 16-bit parameters and at most 64 experts the linear layer, the top-k and the
    softmax are one kernel (two in backward); otherwise the top-k + softmax are.
    """

    def __init__(self, d_model, num_expert, world_size, top_k=2, gate_bias=True):
        super().__init__(num_expert, world_size)
        self.gate = nn.Linear(d_model, self.tot_expert, bias=gate_bias)
        self.top_k = top_k

    def forward(self, inp, return_all_scores=False):
        logits, idx, score = gating.linear_topk_softmax(
            inp.reshape(-1, inp.shape[-1]), self.gate.weight, self.gate.bias, self.top_k)
        logits = logits.view(*inp.shape[:-1], self.tot_expert)
        # The reference installs a zero "dummy" loss so that callers can always add it.
        self.set_loss(torch.zeros(1, device=inp.device, requires_grad=True))
        if return_all_scores:
            return idx, score, logits
        return idx, score
