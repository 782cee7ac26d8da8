r"""Noisy top-k gate of Shazeer et al. (parity: ``fmoe/gates/noisy_gate.py:13-144``)."""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .base_gate import BaseGate

_SQRT2 = math.sqrt(2.0)


def _normal_cdf(x):
    return 0.5 * (1.0 + torch.erf(x / _SQRT2))


def cv_squared(x):
    r"""Squared coefficient of variation ``var/mean²`` (0 for a single element)."""
    if x.numel() <= 1:
        return x.new_zeros(()).float()
    x = x.float()
    return x.var() / (x.mean() ** 2 + 1e-10)


class NoisyGate(BaseGate):
    r"""Logits ``x·w_gate`` plus Gaussian noise of learned scale ``softplus(x·w_noise)+1e-2``
    (training only); top-k with softmax over the selected noisy logits.

    Loss: ``cv²(importance) + cv²(load)`` where *importance* is the summed gate value per
    expert and *load* the (differentiable) probability of each expert being in the top k.
    Returns ids of shape ``[B, k]`` — the reference flattens them, which makes its core
    layer treat the gate as top-1 — and scores of shape ``[B, 1, k]``.
    """

    def __init__(self, d_model, num_expert, world_size, top_k=2):
        super().__init__(num_expert, world_size)
        self.w_gate = nn.Parameter(torch.zeros(d_model, self.tot_expert))
        self.w_noise = nn.Parameter(torch.zeros(d_model, self.tot_expert))
        self.top_k = top_k
        self.noise_epsilon = 1e-2
        self.reset_parameters()

    def reset_parameters(self):
        nn.init.kaiming_uniform_(self.w_gate, a=math.sqrt(5))
        nn.init.kaiming_uniform_(self.w_noise, a=math.sqrt(5))

    def _prob_in_top_k(self, clean, noisy, stddev, noisy_top):
        r"""P(expert stays/enters the top k under fresh noise), per token and expert."""
        # An expert already in the top k must beat the (k+1)-th noisy value; one outside
        # must beat the k-th.
        thr_in = noisy_top[:, self.top_k:self.top_k + 1]
        thr_out = noisy_top[:, self.top_k - 1:self.top_k]
        is_in = noisy > thr_in
        p_in = _normal_cdf((clean - thr_in) / stddev)
        p_out = _normal_cdf((clean - thr_out) / stddev)
        return torch.where(is_in, p_in, p_out)

    def forward(self, inp):
        clean = inp @ self.w_gate
        noisy = clean
        stddev = None
        if self.training:
            stddev = F.softplus(inp @ self.w_noise) + self.noise_epsilon
            noisy = clean + torch.randn_like(clean) * stddev

        m = min(self.top_k + 1, self.tot_expert)
        top_val, top_idx = noisy.topk(m, dim=1)
        k_val, k_idx = top_val[:, :self.top_k], top_idx[:, :self.top_k]
        k_gate = F.softmax(k_val, dim=1)
        gates = torch.zeros_like(noisy).scatter(1, k_idx, k_gate)

        if self.top_k < self.tot_expert and stddev is not None:
            load = self._prob_in_top_k(clean, noisy, stddev, top_val).sum(0)
        else:
            load = (gates > 0).sum(0)
        self.set_loss(cv_squared(gates.sum(0)) + cv_squared(load))
        return k_idx.contiguous(), k_gate.contiguous().unsqueeze(1)
