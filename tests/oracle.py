r"""Brute-force MoE oracles: one token at a time, one expert at a time, plain PyTorch.

They restate the semantics the reference tests check against (``tests/moe.py``): the output
of a token is the score-weighted sum of the outputs of its selected experts; dropped slots
(``-1``) contribute nothing.
"""
import torch
import torch.nn as nn


def moe_mlp_bruteforce(x, idx, score, w1, b1, w2, b2, act):
    r"""``x [B,d]``, ``idx/score [B,k]``, ``w1 [E,h,d]``, ``w2 [E,d,h]`` → ``[B,d]``."""
    out = []
    for t in range(x.shape[0]):
        acc = torch.zeros(w2.shape[1], dtype=x.dtype, device=x.device)
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            if e < 0:
                continue
            h = act(x[t] @ w1[e].t() + b1[e])
            acc = acc + score[t, j] * (h @ w2[e].t() + b2[e])
        out.append(acc)
    return torch.stack(out)


def moe_bruteforce(x, idx, score, experts):
    r"""Arbitrary expert modules called as ``expert(rows, count)``."""
    out = []
    for t in range(x.shape[0]):
        acc = None
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            if e < 0:
                continue
            y = experts[e](x[t:t + 1], torch.tensor([1]))[0] * score[t, j]
            acc = y if acc is None else acc + y
        out.append(acc)
    return torch.stack(out)


class LinearExpert(nn.Module):
    r"""Expert with the ``(rows, count)`` calling convention around a small MLP."""

    def __init__(self, d_model):
        super().__init__()
        self.model = nn.Sequential(nn.Linear(d_model, 2 * d_model), nn.ReLU(),
                                   nn.Linear(2 * d_model, d_model))

    def forward(self, x, _count=None):
        return self.model(x)
