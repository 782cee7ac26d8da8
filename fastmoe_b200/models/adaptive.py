r"""
Adaptive input embedding and adaptive (clustered) softmax for large vocabularies.

The reference's Transformer-XL example uses them for WikiText-103 and One-Billion-Word
(``examples/transformer-xl/mem_transformer.py:464-540`` ``AdaptiveEmbedding``,
``examples/transformer-xl/utils/proj_adaptive_softmax.py`` ``ProjectedAdaptiveLogSoftmax``).
This module is written from the method's definition (Grave et al., "Efficient softmax
approximation for GPUs"; Baevski & Auli, "Adaptive input representations"):

* the vocabulary, sorted by frequency, is cut at ``cutoffs`` into a *shortlist* and tail
  clusters; cluster ``i`` uses an embedding width of ``d_embed / div_val**i`` and a projection
  to / from the model width ``d_proj``;
* the head softmax ranges over the shortlist tokens plus one entry per tail cluster, and
  ``log p(w) = log p_head(cluster(w)) + log p_cluster(w)`` for a tail token.

One parameter layout serves every ``div_val``: per cluster an embedding table, a projection
(absent when the widths agree), an output weight (optionally tied to the table) and a bias.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F


def _cluster_bounds(n_token, cutoffs):
    cuts = [c for c in sorted(set(int(c) for c in cutoffs)) if 0 < c < n_token]
    edges = [0] + cuts + [n_token]
    return list(zip(edges[:-1], edges[1:]))


class AdaptiveEmbedding(nn.Module):
    r"""``forward(tokens [...]) -> [..., d_proj]``, scaled by ``sqrt(d_proj)``."""

    def __init__(self, n_token, d_embed, d_proj, cutoffs=(), div_val=1):
        super().__init__()
        self.n_token, self.d_embed, self.d_proj, self.div_val = n_token, d_embed, d_proj, div_val
        self.bounds = _cluster_bounds(n_token, cutoffs)
        self.emb_scale = d_proj ** 0.5
        self.emb_layers = nn.ModuleList()
        self.emb_projs = nn.ParameterList()
        for i, (lo, hi) in enumerate(self.bounds):
            width = max(1, d_embed // (div_val ** i))
            self.emb_layers.append(nn.Embedding(hi - lo, width))
            # A projection exists whenever the cluster width differs from the model width.
            self.emb_projs.append(nn.Parameter(torch.empty(d_proj, width).normal_(0.0, 0.01))
                                  if width != d_proj else nn.Parameter(torch.empty(0), requires_grad=False))

    def cluster_width(self, i):
        return self.emb_layers[i].embedding_dim

    def forward(self, tokens):
        flat = tokens.reshape(-1)
        out = self.emb_layers[0].weight.new_zeros(flat.numel(), self.d_proj)
        for i, (lo, hi) in enumerate(self.bounds):
            if len(self.bounds) == 1:
                sel, local = None, flat
            else:
                sel = ((flat >= lo) & (flat < hi)).nonzero(as_tuple=True)[0]
                if sel.numel() == 0:
                    continue
                local = flat[sel] - lo
            emb = self.emb_layers[i](local)
            if self.emb_projs[i].numel():
                emb = F.linear(emb, self.emb_projs[i])
            if sel is None:
                out = emb
            else:
                out.index_copy_(0, sel, emb.to(out.dtype))
        return out.view(*tokens.shape, self.d_proj) * self.emb_scale


class ProjectedAdaptiveLogSoftmax(nn.Module):
    r"""``forward(hidden [N, d_proj], target [N]) -> nll [N]``.

    ``tie_weights(embedding)`` shares the output weights with an :class:`AdaptiveEmbedding` of
    the same shape; ``tie_projs`` lists, per cluster, whether the projection is shared too.
    """

    def __init__(self, n_token, d_embed, d_proj, cutoffs=(), div_val=1):
        super().__init__()
        self.n_token, self.d_embed, self.d_proj, self.div_val = n_token, d_embed, d_proj, div_val
        self.bounds = _cluster_bounds(n_token, cutoffs)
        self.n_clusters = len(self.bounds) - 1
        self.shortlist = self.bounds[0][1]
        width0 = max(1, d_embed)
        if self.n_clusters > 0:
            self.cluster_weight = nn.Parameter(torch.zeros(self.n_clusters, width0))
            self.cluster_bias = nn.Parameter(torch.zeros(self.n_clusters))
        self.out_layers = nn.ModuleList()
        self.out_projs = nn.ParameterList()
        for i, (lo, hi) in enumerate(self.bounds):
            width = max(1, d_embed // (div_val ** i))
            self.out_layers.append(nn.Linear(width, hi - lo))
            self.out_projs.append(nn.Parameter(torch.empty(d_proj, width).normal_(0.0, 0.01))
                                  if width != d_proj else nn.Parameter(torch.empty(0), requires_grad=False))

    def tie_weights(self, embedding, tie_projs=None):
        assert [tuple(b) for b in embedding.bounds] == [tuple(b) for b in self.bounds]
        for i in range(len(self.bounds)):
            self.out_layers[i].weight = embedding.emb_layers[i].weight
            if tie_projs is not None and i < len(tie_projs) and tie_projs[i] and self.out_projs[i].numel():
                self.out_projs[i] = embedding.emb_projs[i]

    def _logits(self, hidden, i, extra_w=None, extra_b=None):
        proj = self.out_projs[i]
        h = F.linear(hidden, proj.t()) if proj.numel() else hidden
        w, b = self.out_layers[i].weight, self.out_layers[i].bias
        if extra_w is not None:
            w = torch.cat([w, extra_w], 0)
            b = torch.cat([b, extra_b], 0)
        return F.linear(h, w, b)

    def _head_logprob(self, hidden):
        if self.n_clusters > 0:
            logit = self._logits(hidden, 0, self.cluster_weight, self.cluster_bias)
        else:
            logit = self._logits(hidden, 0)
        return F.log_softmax(logit.float(), dim=-1)

    def log_prob(self, hidden):
        r"""Full ``[N, n_token]`` log-probabilities (evaluation and tests)."""
        head = self._head_logprob(hidden)
        parts = [head[:, :self.shortlist]]
        for i in range(1, len(self.bounds)):
            tail = F.log_softmax(self._logits(hidden, i).float(), dim=-1)
            parts.append(head[:, self.shortlist + i - 1:self.shortlist + i] + tail)
        return torch.cat(parts, dim=-1)

    def forward(self, hidden, target):
        assert hidden.shape[0] == target.shape[0]
        head = self._head_logprob(hidden)
        if self.n_clusters == 0:
            return -head.gather(1, target[:, None]).squeeze(1)
        nll = head.new_zeros(target.shape[0])
        for i, (lo, hi) in enumerate(self.bounds):
            sel = ((target >= lo) & (target < hi)).nonzero(as_tuple=True)[0]
            if sel.numel() == 0:
                continue
            local = (target[sel] - lo)[:, None]
            if i == 0:
                lp = head[sel].gather(1, local).squeeze(1)
            else:
                tail = F.log_softmax(self._logits(hidden[sel], i).float(), dim=-1)
                lp = head[sel, self.shortlist + i - 1] + tail.gather(1, local).squeeze(1)
            nll.index_copy_(0, sel, -lp)
        return nll
