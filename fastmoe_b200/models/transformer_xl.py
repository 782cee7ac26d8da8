r"""
Transformer-XL language model with MoE feed-forward blocks.

Covers what the reference's example model provides (``examples/transformer-xl/mem_transformer.py``):
segment-level recurrence with a memory of ``mem_len`` cached hidden states per layer
(``:222-231,675-696`` there), relative positional attention with the ``_rel_shift`` trick
(``:195-208``), and the MoE position-wise feed-forward ``CustomizedMoEPositionwiseFF``
(``:379-409``): ``FMoETransformerMLP`` with ``Sequential(ReLU, Dropout)`` between the expert
linears, residual connection and LayerNorm.  Unlike the example — a single process with
``nn.DataParallel`` and ``world_size=1`` — the MoE blocks take ``world_size`` / ``moe_group`` and
run expert-parallel.  Written from the paper's equations; inputs are ``[seq, batch]``.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from ..transformer import FMoETransformerMLP
from .adaptive import AdaptiveEmbedding, ProjectedAdaptiveLogSoftmax
from .sampled_softmax import LogUniformSampler, sampled_softmax_nll


class PositionalEmbedding(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.register_buffer("inv_freq", 1.0 / (10000 ** (torch.arange(0.0, d, 2.0) / d)), persistent=False)

    def forward(self, pos_seq):
        ang = torch.outer(pos_seq, self.inv_freq.to(pos_seq.dtype))
        return torch.cat([ang.sin(), ang.cos()], dim=-1)             # [klen, d]


class PositionwiseFF(nn.Module):
    r"""Dense feed-forward block (the non-MoE baseline)."""

    def __init__(self, d_model, d_inner, dropout, pre_lnorm=False):
        super().__init__()
        self.core = nn.Sequential(nn.Linear(d_model, d_inner), nn.ReLU(inplace=True), nn.Dropout(dropout),
                                  nn.Linear(d_inner, d_model), nn.Dropout(dropout))
        self.layer_norm = nn.LayerNorm(d_model)
        self.pre_lnorm = pre_lnorm

    def forward(self, x):
        if self.pre_lnorm:
            return x + self.core(self.layer_norm(x))
        return self.layer_norm(x + self.core(x))


class MoEPositionwiseFF(FMoETransformerMLP):
    r"""MoE feed-forward block: residual + LayerNorm around an expert-parallel MLP."""

    def __init__(self, d_model, d_inner, dropout, pre_lnorm=False, moe_num_expert=64, moe_top_k=2,
                 world_size=1, moe_group=None, gate=None):
        kwargs = {} if gate is None else {"gate": gate}
        super().__init__(num_expert=moe_num_expert, d_model=d_model, d_hidden=d_inner, top_k=moe_top_k,
                         activation=nn.Sequential(nn.ReLU(), nn.Dropout(dropout)),
                         world_size=world_size, moe_group=moe_group, **kwargs)
        self.pre_lnorm = pre_lnorm
        self.layer_norm = nn.LayerNorm(d_model)
        self.dropout = nn.Dropout(dropout)

    def forward(self, x):
        if self.pre_lnorm:
            return x + self.dropout(super().forward(self.layer_norm(x)))
        return self.layer_norm(x + self.dropout(super().forward(x)))


class RelMultiHeadAttn(nn.Module):
    r"""Multi-head attention with Transformer-XL relative positions and a memory of past states."""

    def __init__(self, n_head, d_model, d_head, dropout, dropatt=0.0, pre_lnorm=False):
        super().__init__()
        self.n_head, self.d_head = n_head, d_head
        self.qkv_net = nn.Linear(d_model, 3 * n_head * d_head, bias=False)
        self.r_net = nn.Linear(d_model, n_head * d_head, bias=False)
        self.o_net = nn.Linear(n_head * d_head, d_model, bias=False)
        self.drop = nn.Dropout(dropout)
        self.dropatt = nn.Dropout(dropatt)
        self.layer_norm = nn.LayerNorm(d_model)
        self.scale = 1.0 / (d_head ** 0.5)
        self.pre_lnorm = pre_lnorm

    @staticmethod
    def _rel_shift(x):
        # x: [qlen, klen, batch, head]: shift row i left by (qlen - 1 - i)
        q, k = x.shape[0], x.shape[1]
        pad = x.new_zeros((q, 1) + tuple(x.shape[2:]))
        rest = tuple(x.shape[2:])
        x = torch.cat([pad, x], dim=1).view((k + 1, q) + rest)
        return x[1:].reshape((q, k) + rest)

    def forward(self, w, r, r_w_bias, r_r_bias, attn_mask=None, mems=None):
        qlen, bsz = w.shape[0], w.shape[1]
        cat = w if mems is None or mems.numel() == 0 else torch.cat([mems.to(w.dtype), w], 0)
        heads = self.qkv_net(self.layer_norm(cat) if self.pre_lnorm else cat)
        q, k, v = torch.chunk(heads, 3, dim=-1)
        q = q[-qlen:]
        klen = k.shape[0]
        q = q.view(qlen, bsz, self.n_head, self.d_head)
        k = k.view(klen, bsz, self.n_head, self.d_head)
        v = v.view(klen, bsz, self.n_head, self.d_head)
        r_k = self.r_net(r).view(klen, self.n_head, self.d_head)

        ac = torch.einsum("ibnd,jbnd->ijbn", q + r_w_bias, k)
        bd = self._rel_shift(torch.einsum("ibnd,jnd->ijbn", q + r_r_bias, r_k))
        score = (ac + bd) * self.scale
        if attn_mask is not None:
            score = score.float().masked_fill(attn_mask[:, :, None, None], float("-inf")).type_as(score)
        prob = self.dropatt(F.softmax(score, dim=1))
        vec = torch.einsum("ijbn,jbnd->ibnd", prob, v).reshape(qlen, bsz, self.n_head * self.d_head)
        out = self.drop(self.o_net(vec))
        return w + out if self.pre_lnorm else self.layer_norm(w + out)


class DecoderLayer(nn.Module):
    def __init__(self, n_head, d_model, d_head, d_inner, dropout, dropatt, pre_lnorm, moe, moe_kwargs):
        super().__init__()
        self.dec_attn = RelMultiHeadAttn(n_head, d_model, d_head, dropout, dropatt, pre_lnorm)
        if moe:
            self.pos_ff = MoEPositionwiseFF(d_model, d_inner, dropout, pre_lnorm, **moe_kwargs)
        else:
            self.pos_ff = PositionwiseFF(d_model, d_inner, dropout, pre_lnorm)

    def forward(self, x, r, r_w_bias, r_r_bias, attn_mask, mems):
        return self.pos_ff(self.dec_attn(x, r, r_w_bias, r_r_bias, attn_mask, mems))


class MemTransformerLM(nn.Module):
    r"""``forward(data, target, *mems) -> [loss [tgt_len, batch]] + new_mems``.

    Keyword arguments follow the example model: ``n_token, n_layer, n_head, d_model, d_head,
    d_inner, dropout, dropatt, tie_weight, pre_lnorm, tgt_len, ext_len, mem_len, same_length,
    clamp_len, moe, moe_num_expert, moe_top_k`` plus ``world_size`` / ``moe_group`` / ``gate``.
    ``d_embed`` / ``cutoffs`` / ``div_val`` / ``tie_projs`` select the adaptive embedding and
    adaptive softmax used for large vocabularies (``--adaptive`` in the training script); with
    no cut-offs and ``d_embed == d_model`` a plain embedding and a plain (tied) output layer
    are used.  ``sample_softmax=N`` trains against ``N`` log-uniform negatives
    (:mod:`fastmoe_b200.models.sampled_softmax`); evaluation always uses the full softmax.
    """

    def __init__(self, n_token, n_layer, n_head, d_model, d_head, d_inner, dropout=0.1, dropatt=0.0,
                 tie_weight=True, pre_lnorm=False, tgt_len=512, ext_len=0, mem_len=512,
                 same_length=False, clamp_len=-1, moe=False, moe_num_expert=64, moe_top_k=2,
                 world_size=1, moe_group=None, gate=None, d_embed=None, cutoffs=(), div_val=1,
                 tie_projs=(), sample_softmax=-1):
        super().__init__()
        self.n_token, self.n_layer, self.d_model = n_token, n_layer, d_model
        d_embed = d_model if d_embed is None or d_embed <= 0 else d_embed
        self.adaptive = bool(cutoffs) or d_embed != d_model or div_val != 1
        self.tgt_len, self.ext_len, self.mem_len = tgt_len, ext_len, mem_len
        self.same_length, self.clamp_len = same_length, clamp_len
        if self.adaptive:
            self.word_emb = AdaptiveEmbedding(n_token, d_embed, d_model, cutoffs, div_val)
            self.emb_scale = 1.0   # the adaptive embedding applies sqrt(d_model) itself
        else:
            self.word_emb = nn.Embedding(n_token, d_model)
            self.emb_scale = d_model ** 0.5
        self.drop = nn.Dropout(dropout)
        self.pos_emb = PositionalEmbedding(d_model)
        self.r_w_bias = nn.Parameter(torch.zeros(n_head, d_head))
        self.r_r_bias = nn.Parameter(torch.zeros(n_head, d_head))
        moe_kwargs = dict(moe_num_expert=moe_num_expert, moe_top_k=moe_top_k, world_size=world_size,
                          moe_group=moe_group, gate=gate)
        self.layers = nn.ModuleList([
            DecoderLayer(n_head, d_model, d_head, d_inner, dropout, dropatt, pre_lnorm, moe, moe_kwargs)
            for _ in range(n_layer)])
        if self.adaptive:
            self.crit = ProjectedAdaptiveLogSoftmax(n_token, d_embed, d_model, cutoffs, div_val)
            self.out_layer = None
        else:
            self.crit = None
            self.out_layer = nn.Linear(d_model, n_token)
        self.apply(self._init)
        # --sample_softmax N: train against N log-uniform negatives instead of the full softmax
        self.sample_softmax = sample_softmax
        self.sampler = None
        if sample_softmax > 0:
            assert not self.adaptive, "sampled softmax works on the plain output layer"
            self.sampler = LogUniformSampler(n_token, sample_softmax)
        if tie_weight:
            if self.adaptive:
                self.crit.tie_weights(self.word_emb, tie_projs)
            else:
                self.out_layer.weight = self.word_emb.weight

    @staticmethod
    def _init(m):
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, 0.0, 0.02)
            if m.bias is not None:
                nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, 0.0, 0.02)

    def reset_length(self, tgt_len, ext_len, mem_len):
        self.tgt_len, self.ext_len, self.mem_len = tgt_len, ext_len, mem_len

    def init_mems(self, device=None, dtype=None):
        if self.mem_len <= 0:
            return []
        p = self.r_w_bias
        return [torch.empty(0, dtype=dtype or p.dtype, device=device or p.device)
                for _ in range(self.n_layer + 1)]

    def _update_mems(self, hids, mems, qlen, mlen):
        if not mems:
            return []
        with torch.no_grad():
            end = mlen + max(0, qlen - self.ext_len)
            beg = max(0, end - self.mem_len)
            return [torch.cat([m.to(h.dtype), h], 0)[beg:end].detach() if m.numel() else h[beg:end].detach()
                    for m, h in zip(mems, hids)]

    def _forward(self, data, mems):
        qlen = data.shape[0]
        mlen = mems[0].shape[0] if mems and mems[0].numel() else 0
        klen = mlen + qlen
        x = self.drop(self.word_emb(data) * self.emb_scale)
        ones = torch.ones(qlen, klen, dtype=torch.bool, device=data.device)
        mask = torch.triu(ones, diagonal=1 + mlen)
        if self.same_length:
            mask = mask | torch.tril(ones, diagonal=mlen - qlen if self.mem_len > 0 else 0 - qlen)
        pos_seq = torch.arange(klen - 1, -1, -1.0, device=data.device, dtype=x.dtype)
        if self.clamp_len > 0:
            pos_seq = pos_seq.clamp(max=self.clamp_len)
        r = self.drop(self.pos_emb(pos_seq).to(x.dtype))
        hids = [x]
        for i, layer in enumerate(self.layers):
            mem_i = mems[i] if mems else None
            x = layer(x, r, self.r_w_bias, self.r_r_bias, mask, mem_i)
            hids.append(x)
        return self.drop(x), self._update_mems(hids, mems, qlen, mlen)

    def forward(self, data, target, *mems):
        mems = list(mems) if mems else self.init_mems(device=data.device)
        hidden, new_mems = self._forward(data, mems)
        tgt_len = target.shape[0]
        pred = hidden[-tgt_len:]
        if self.adaptive:
            loss = self.crit(pred.reshape(-1, pred.shape[-1]), target.reshape(-1)).view(tgt_len, -1)
        elif self.sampler is not None and self.training:
            loss = sampled_softmax_nll(self.out_layer.weight, self.out_layer.bias,
                                       pred.reshape(-1, pred.shape[-1]), target.reshape(-1),
                                       self.sampler).view(tgt_len, -1)
        else:
            logits = self.out_layer(pred)
            loss = F.cross_entropy(logits.float().view(-1, self.n_token), target.reshape(-1),
                                   reduction="none").view(tgt_len, -1)
        return [loss] + new_mems

    def balance_losses(self):
        out = []
        for layer in self.layers:
            gate = getattr(layer.pos_ff, "gate", None)
            if gate is not None and gate.has_loss:
                out.append(gate.get_loss(clear=False).reshape(1))
        return out
