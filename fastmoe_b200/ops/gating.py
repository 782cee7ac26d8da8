r"""
Gate math: top-k selection with softmax over the selected logits.

Parity: the ``topk`` → ``softmax`` sequence of ``fmoe/gates/naive_gate.py:31-38`` (ATen ops
in the reference).  On a GPU one kernel reads each logits row once, keeps the k largest in
registers, writes ids and probabilities, and a second small kernel applies the softmax
Jacobian in backward and scatters the result into the dense logits gradient.
"""
import torch
from torch.autograd import Function

from . import native

MAX_FUSED_K = 8
MAX_FUSED_EXPERTS = 4096


def _topk_softmax_torch(logits, k):
    val, idx = torch.topk(logits, k=k, dim=-1, largest=True, sorted=True)
    return idx, torch.softmax(val, dim=-1)


class _TopkSoftmax(Function):
    @staticmethod
    def forward(ctx, logits, k):
        idx, score = native.get().gate_topk_softmax(logits.contiguous(), int(k))
        ctx.save_for_backward(idx, score)
        ctx.shape = logits.shape
        ctx.mark_non_differentiable(idx)
        return idx, score

    @staticmethod
    def backward(ctx, _grad_idx, grad_score):
        idx, score = ctx.saved_tensors
        grad_logits = native.get().gate_topk_softmax_bwd(
            grad_score.contiguous(), idx, score, int(ctx.shape[-1]))
        return grad_logits, None


def topk_softmax(logits, k):
    r"""``(idx int64 [B,k], prob [B,k])``: the k largest logits per row (descending) and their softmax."""
    if (logits.is_cuda and k <= MAX_FUSED_K and logits.shape[-1] <= MAX_FUSED_EXPERTS
            and logits.dtype in (torch.float32, torch.bfloat16, torch.float16)):
        return _TopkSoftmax.apply(logits, k)
    return _topk_softmax_torch(logits, k)
