r"""
Sampled softmax with a log-uniform candidate sampler, for training with very large vocabularies.

The reference's Transformer-XL example has it behind ``--sample_softmax N``
(``examples/transformer-xl/utils/log_uniform_sampler.py``, used at
``examples/transformer-xl/mem_transformer.py:748-757``).  Written here from the method's
definition (Jean et al., "On using very large target vocabulary for neural machine
translation"; the log-uniform sampler of word2vec / TensorFlow): with the vocabulary sorted by
frequency, class ``k`` is proposed with probability
``P(k) = (log(k + 2) - log(k + 1)) / log(range_max + 1)``; a batch shares ``n_sample`` distinct
negatives drawn with ``2 * n_sample`` tries, every logit is corrected by minus the log of the
expected number of times its class is proposed, and negatives that coincide with a row's
target are masked.
"""
import math

import torch
import torch.nn.functional as F


class LogUniformSampler:
    r"""``sample(labels) -> (true_log_q, sample_log_q, negatives)``."""

    def __init__(self, range_max, n_sample, generator=None):
        self.range_max, self.n_sample = int(range_max), int(n_sample)
        self.generator = generator
        k = torch.arange(self.range_max, dtype=torch.float64)
        self.prob = ((torch.log(k + 2.0) - torch.log(k + 1.0)) / math.log(self.range_max + 1.0))
        n_tries = 2 * self.n_sample
        # expected number of times a class appears among n_tries draws, counted once (unique)
        self.log_q = torch.log(-torch.expm1(n_tries * torch.log1p(-self.prob))).float()

    def sample(self, labels):
        n_tries = 2 * self.n_sample
        draws = torch.multinomial(self.prob, n_tries, replacement=True, generator=self.generator)
        negatives = torch.unique(draws).to(labels.device)
        log_q = self.log_q.to(labels.device)
        return log_q[labels], log_q[negatives], negatives


def sampled_softmax_nll(weight, bias, hidden, labels, sampler):
    r"""Negative log-likelihood of ``labels`` under a softmax over {target} ∪ negatives.

    ``weight [n_token, d]`` / ``bias [n_token]``: the output layer; ``hidden [N, d]``;
    ``labels [N]``.  Returns ``[N]``.
    """
    true_log_q, samp_log_q, negatives = sampler.sample(labels)
    true_w, true_b = weight[labels], bias[labels]
    samp_w, samp_b = weight[negatives], bias[negatives]
    true_logit = (hidden * true_w).sum(-1) + true_b - true_log_q.to(hidden.dtype)
    samp_logit = hidden @ samp_w.t() + samp_b - samp_log_q.to(hidden.dtype)
    hit = labels[:, None] == negatives[None, :]
    samp_logit = samp_logit.masked_fill(hit, -1e30)
    logits = torch.cat([true_logit[:, None], samp_logit], dim=1).float()
    return -F.log_softmax(logits, dim=-1)[:, 0]
