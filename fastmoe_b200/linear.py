r"""
Grouped ("parallel") linear layer: one weight matrix per local expert.

Parity: ``fmoe/linear.py`` — the autograd function ``MOELinear`` (``:12-36``) and the module
``FMoELinear`` (``:40-91``) with the parameter layout ``weight [num_expert, out_feat, in_feat]``,
``bias [num_expert, out_feat]`` (zero at start), ``nn.Linear``'s weight distribution, and the
``rank`` argument that is only reported by ``repr``.

The rows of the input are grouped by expert and ``fwd_expert_count[e]`` of them belong to
expert ``e``.  On a B200 the forward, input-gradient and weight-gradient GEMMs and the bias
gradient are tcgen05 kernels over all experts at once (:mod:`fastmoe_b200.ops.grouped_gemm`);
the reference loops over the experts on the host with one cuBLAS call each
(``cuda/parallel_linear.cuh:56-163``).
"""
import math

import torch
from torch import nn
from torch.autograd import Function

from .ops import api as _ops


class MOELinear(Function):
    r"""``out[rows_e] = inp[rows_e] @ weight[e].T (+ bias[e])`` for every local expert ``e``."""

    @staticmethod
    def forward(ctx, global_input_buf, fwd_expert_count, weight, bias=None):
        ctx.save_for_backward(global_input_buf, fwd_expert_count, weight, bias)
        return _ops.linear_forward(global_input_buf, fwd_expert_count, weight, bias)

    @staticmethod
    def backward(ctx, grad_out):
        rows, counts, weight, bias = ctx.saved_tensors
        d_rows, d_weight, d_bias = _ops.linear_backward(grad_out.contiguous(), rows, counts, weight, bias)
        # one gradient slot per forward argument: (rows, counts, weight, bias)
        return d_rows, None, d_weight, (d_bias if torch.is_tensor(bias) else None)


class FMoELinear(nn.Module):
    r"""``num_expert`` independent linear maps ``in_feat → out_feat`` evaluated in one call:
    ``layer(inp, fwd_expert_count)``."""

    def __init__(self, num_expert: int, in_feat: int, out_feat: int, bias: bool = True,
                 rank: int = 0):
        super().__init__()
        self.num_expert, self.in_feat, self.out_feat, self.rank = num_expert, in_feat, out_feat, rank
        self.weight = nn.Parameter(torch.empty(num_expert, out_feat, in_feat))
        self.register_parameter("bias", nn.Parameter(torch.zeros(num_expert, out_feat)) if bias else None)
        self.reset_parameters()

    def reset_parameters(self):
        r"""Weights as ``nn.Linear`` draws them (per expert matrix); biases are left at zero."""
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))

    def forward(self, inp, fwd_expert_count):
        return MOELinear.apply(inp.type_as(self.weight), fwd_expert_count, self.weight, self.bias)

    def extra_repr(self) -> str:
        fields = (("num_expert", self.num_expert), ("in_features", self.in_feat),
                  ("out_features", self.out_feat), ("bias", self.bias is not None), ("rank", self.rank))
        return ", ".join("%s=%s" % kv for kv in fields)
