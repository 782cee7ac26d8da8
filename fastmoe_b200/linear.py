r"""
Grouped ("parallel") linear layer: one weight matrix per local expert.

Parity: ``fmoe/linear.py`` — ``MOELinear`` (``:12-36``) and ``FMoELinear`` (``:40-91``),
including the parameter layout ``weight [num_expert, out_feat, in_feat]``,
``bias [num_expert, out_feat]`` (zero-initialised), kaiming-uniform(a=√5) weight init and
the unused ``rank`` argument that only shows up in ``extra_repr``.

On a B200 the three GEMMs (forward, input gradient, weight gradient) and the bias
gradient are tcgen05 kernels that read the expert row offsets from device memory
(:mod:`fastmoe_b200.ops.grouped_gemm`); the reference instead loops over experts on the
host, one cuBLAS call each, with a stream synchronisation before and after
(``cuda/parallel_linear.cuh:56-163``).
"""
import math

import torch
import torch.nn as nn
from torch.autograd import Function

from .ops import api as _ops


class MOELinear(Function):
    r"""``y[rows of expert e] = x[rows of expert e] @ weight[e].T + bias[e]``."""

    @staticmethod
    def forward(ctx, global_input_buf, fwd_expert_count, weight, bias=None):
        out = _ops.linear_forward(global_input_buf, fwd_expert_count, weight, bias)
        ctx.save_for_backward(global_input_buf, fwd_expert_count, weight, bias)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        inp, fwd_expert_count, weight, bias = ctx.saved_tensors
        grad_in, grad_w, grad_b = _ops.linear_backward(
            grad_out.contiguous(), inp, fwd_expert_count, weight, bias)
        if not torch.is_tensor(bias):
            grad_b = None
        return grad_in, None, grad_w, grad_b


class FMoELinear(nn.Module):
    r"""A linear layer holding ``num_expert`` independent weight matrices.

    ``forward(inp, fwd_expert_count)``: ``inp`` rows are grouped by expert and
    ``fwd_expert_count[e]`` rows belong to expert ``e``.
    """

    def __init__(self, num_expert: int, in_feat: int, out_feat: int, bias: bool = True,
                 rank: int = 0):
        super().__init__()
        self.num_expert = num_expert
        self.in_feat = in_feat
        self.out_feat = out_feat
        self.rank = rank
        self.weight = nn.Parameter(torch.empty(num_expert, out_feat, in_feat))
        if bias:
            self.bias = nn.Parameter(torch.zeros(num_expert, out_feat))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self):
        # Same distribution as torch.nn.Linear's weight; the bias stays at zero.
        torch.nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))

    def forward(self, inp, fwd_expert_count):
        return MOELinear.apply(inp.type_as(self.weight), fwd_expert_count, self.weight, self.bias)

    def extra_repr(self) -> str:
        return "num_expert={}, in_features={}, out_features={}, bias={}, rank={}".format(
            self.num_expert, self.in_feat, self.out_feat, self.bias is not None, self.rank)
