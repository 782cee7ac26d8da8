r"""
A Megatron-shaped GPT for the ``fmoefy`` path.

The module tree mirrors what ``fmoe/megatron/layers.py:196-222`` walks in Megatron-LM v2.5 /
v3.0.2 — ``model.language_model.encoder.layers[i].mlp`` — (and ``language_model.transformer``
is an alias of the same stack for the v2.2 layout), the MLP returns ``(output, bias)`` like
Megatron's ``ParallelMLP``, and the model offers ``state_dict_for_save_checkpoint`` and
``set_input_tensor``.  Attention uses ``scaled_dot_product_attention``; it is outside the MoE
paths this project rewrites.
"""
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class GPTConfig:
    hidden_size: int = 1024
    num_layers: int = 24
    num_attention_heads: int = 16
    ffn_hidden_size: int = 4096
    vocab_size: int = 50257
    max_position_embeddings: int = 1024
    init_method_std: float = 0.02
    layernorm_epsilon: float = 1e-5
    hidden_dropout: float = 0.0
    attention_dropout: float = 0.0


class ParallelMLP(nn.Module):
    r"""Dense feed-forward block with Megatron's calling convention: returns ``(output, bias)``."""

    def __init__(self, cfg):
        super().__init__()
        self.dense_h_to_4h = nn.Linear(cfg.hidden_size, cfg.ffn_hidden_size)
        self.dense_4h_to_h = nn.Linear(cfg.ffn_hidden_size, cfg.hidden_size)

    def forward(self, x):
        y = self.dense_4h_to_h(F.gelu(self.dense_h_to_4h(x)))
        return y, torch.zeros(y.shape[-1], dtype=y.dtype, device=y.device)


class ParallelAttention(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.heads = cfg.num_attention_heads
        self.query_key_value = nn.Linear(cfg.hidden_size, 3 * cfg.hidden_size)
        self.dense = nn.Linear(cfg.hidden_size, cfg.hidden_size)
        self.dropout = cfg.attention_dropout

    def forward(self, x):
        # x: [seq, batch, hidden]
        s, b, h = x.shape
        qkv = self.query_key_value(x).view(s, b, 3, self.heads, h // self.heads)
        q, k, v = (qkv[:, :, i].permute(1, 2, 0, 3) for i in range(3))    # [b, heads, s, dh]
        ctx = F.scaled_dot_product_attention(q, k, v, is_causal=True,
                                             dropout_p=self.dropout if self.training else 0.0)
        return self.dense(ctx.permute(2, 0, 1, 3).reshape(s, b, h))


class ParallelTransformerLayer(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.input_layernorm = nn.LayerNorm(cfg.hidden_size, eps=cfg.layernorm_epsilon)
        self.self_attention = ParallelAttention(cfg)
        self.post_attention_layernorm = nn.LayerNorm(cfg.hidden_size, eps=cfg.layernorm_epsilon)
        self.mlp = ParallelMLP(cfg)
        self.hidden_dropout = cfg.hidden_dropout

    def forward(self, x):
        x = x + F.dropout(self.self_attention(self.input_layernorm(x)), self.hidden_dropout, self.training)
        out, bias = self.mlp(self.post_attention_layernorm(x))
        return x + F.dropout(out + bias, self.hidden_dropout, self.training)


class ParallelTransformer(nn.Module):
    def __init__(self, cfg, num_layers=None):
        super().__init__()
        n = cfg.num_layers if num_layers is None else num_layers
        self.layers = nn.ModuleList([ParallelTransformerLayer(cfg) for _ in range(n)])
        self.final_layernorm = nn.LayerNorm(cfg.hidden_size, eps=cfg.layernorm_epsilon)
        self.input_tensor = None

    def set_input_tensor(self, t):
        self.input_tensor = t

    def forward(self, x, final_norm=True):
        if self.input_tensor is not None:
            x = self.input_tensor
        for layer in self.layers:
            x = layer(x)
        return self.final_layernorm(x) if final_norm else x


class Embedding(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.word_embeddings = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.position_embeddings = nn.Embedding(cfg.max_position_embeddings, cfg.hidden_size)

    def forward(self, tokens):
        # tokens: [batch, seq] -> [seq, batch, hidden]
        pos = torch.arange(tokens.shape[1], device=tokens.device).unsqueeze(0)
        return (self.word_embeddings(tokens) + self.position_embeddings(pos)).transpose(0, 1).contiguous()


class TransformerLanguageModel(nn.Module):
    r"""``embedding`` + ``encoder`` (= ``transformer``, the older attribute name)."""

    def __init__(self, cfg, pre_process=True, post_process=True, num_layers=None):
        super().__init__()
        self.pre_process, self.post_process = pre_process, post_process
        self.embedding = Embedding(cfg) if pre_process else None
        self.encoder = ParallelTransformer(cfg, num_layers)
        self.decoder = None

    @property
    def transformer(self):
        return self.encoder

    def forward(self, tokens_or_hidden):
        x = self.embedding(tokens_or_hidden) if self.pre_process else tokens_or_hidden
        return self.encoder(x, final_norm=self.post_process)


class GPTModel(nn.Module):
    r"""Decoder-only LM; ``forward(tokens, labels)`` returns the mean token cross-entropy."""

    def __init__(self, cfg, pre_process=True, post_process=True, num_layers=None):
        super().__init__()
        self.cfg = cfg
        self.pre_process, self.post_process = pre_process, post_process
        self.language_model = TransformerLanguageModel(cfg, pre_process, post_process, num_layers)
        if post_process and not pre_process:
            self.output_embeddings = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.apply(self._init)

    def _init(self, m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, mean=0.0, std=self.cfg.init_method_std)
        if isinstance(m, nn.Linear) and m.bias is not None:
            nn.init.zeros_(m.bias)

    def set_input_tensor(self, t):
        self.language_model.encoder.set_input_tensor(t)

    def output_weight(self):
        if self.pre_process:
            return self.language_model.embedding.word_embeddings.weight
        return self.output_embeddings.weight

    def forward(self, tokens, labels=None):
        hidden = self.language_model(tokens)                       # [seq, batch, hidden]
        if not self.post_process:
            return hidden
        logits = F.linear(hidden, self.output_weight())            # [seq, batch, vocab]
        if labels is None:
            return logits.transpose(0, 1)
        return F.cross_entropy(logits.float().view(-1, logits.shape[-1]),
                               labels.transpose(0, 1).reshape(-1))

    def state_dict_for_save_checkpoint(self, destination=None, prefix="", keep_vars=False):
        return self.state_dict(destination=destination, prefix=prefix, keep_vars=keep_vars)

    def balance_losses(self):
        r"""Balance losses left by the gates of fmoefy-ed layers in the last forward."""
        out = []
        for layer in self.language_model.encoder.layers:
            gate = getattr(layer.mlp, "gate", None)
            if gate is not None and gate.has_loss:
                out.append(gate.get_loss(clear=False).reshape(1))
        return out


def gpt_flops_per_token(cfg, top_k=1, moe_hidden=None):
    r"""Forward+backward model FLOPs per token (attention included), for throughput reports."""
    h, s = cfg.hidden_size, cfg.max_position_embeddings
    ffn = (moe_hidden if moe_hidden is not None else cfg.ffn_hidden_size) * top_k
    per_layer = 2 * (4 * h * h + 2 * h * ffn) + 4 * s * h
    return 3 * (cfg.num_layers * per_layer + 2 * h * cfg.vocab_size)
