r"""CPU tier: the MoE layer against brute-force oracles (world_size = 1)."""
import pytest
import torch
import torch.nn as nn

from fastmoe_b200 import FMoE, FMoETransformerMLP
from fastmoe_b200.gates import NaiveGate
from oracle import LinearExpert, moe_bruteforce, moe_mlp_bruteforce


def _grads(params):
    return [p.grad.clone() for p in params]


def test_config1_transformer_mlp_matches_bruteforce():
    r"""d_model=16, d_hidden=32, 4 experts, NaiveGate top-2, GELU, 64 tokens, fp32, seed 0."""
    torch.manual_seed(0)
    moe = FMoETransformerMLP(num_expert=4, d_model=16, d_hidden=32, world_size=1, top_k=2,
                             gate=NaiveGate, activation=nn.GELU())
    x = torch.randn(64, 16, requires_grad=True)
    y = moe(x)
    y.sum().backward()
    gx = x.grad.clone()
    gp = _grads(moe.parameters())
    moe.zero_grad()

    x2 = x.detach().clone().requires_grad_(True)
    logits = moe.gate.gate(x2)
    val, idx = torch.topk(logits, 2, dim=-1)
    score = torch.softmax(val, dim=-1)
    e = moe.experts
    ref = moe_mlp_bruteforce(x2, idx, score, e.htoh4.weight, e.htoh4.bias,
                             e.h4toh.weight, e.h4toh.bias, nn.GELU())
    ref.sum().backward()
    assert torch.allclose(y, ref, atol=1e-5)
    assert torch.allclose(gx, x2.grad, atol=1e-5)
    for a, p in zip(gp, moe.parameters()):
        assert torch.allclose(a, p.grad, atol=1e-4), "param grad mismatch"


@pytest.mark.parametrize("num_expert,top_k", [(4, 2), (8, 3), (3, 1)])
def test_general_path_arbitrary_experts(num_expert, top_k):
    torch.manual_seed(1)
    d = 8
    moe = FMoE(num_expert=num_expert, d_model=d, world_size=1, top_k=top_k, expert=LinearExpert)
    x = torch.randn(20, d, requires_grad=True)
    y = moe(x)
    y.sum().backward()
    gx = x.grad.clone()
    gp = _grads(moe.parameters())
    moe.zero_grad()

    x2 = x.detach().clone().requires_grad_(True)
    val, idx = torch.topk(moe.gate.gate(x2), top_k, dim=-1)
    score = torch.softmax(val, dim=-1)
    ref = moe_bruteforce(x2, idx, score, moe.experts)
    ref.sum().backward()
    assert torch.allclose(y, ref, atol=1e-5)
    assert torch.allclose(gx, x2.grad, atol=1e-5)
    for a, p in zip(gp, moe.parameters()):
        if p.grad is None:
            assert float(a.abs().max()) == 0.0
        else:
            assert torch.allclose(a, p.grad, atol=1e-4)
