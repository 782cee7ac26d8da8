r"""GPU tier: whole layers against fp32 PyTorch oracles (the matrix of the reference's
``tests/test_numerical.py``: expert counts, top-k, dtypes; plus gates and pytree inputs)."""
import pytest
import torch
import torch.nn as nn

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _fp32_leaves(moe):
    e = moe.experts
    return [t.detach().float().requires_grad_(True)
            for t in (e.htoh4.weight, e.htoh4.bias, e.h4toh.weight, e.h4toh.bias)]


def _dense_reference(moe, x32, idx, score32, leaves=None):
    r"""fp32 evaluation of an FMoETransformerMLP with given routing (vectorised per expert)."""
    e = moe.experts
    w1, b1, w2, b2 = leaves if leaves is not None else _fp32_leaves(moe)
    out = torch.zeros_like(x32)
    for j in range(idx.shape[1]):
        for ex in range(w1.shape[0]):
            m = idx[:, j] == ex
            if m.any():
                h = e.activation(x32[m] @ w1[ex].t() + b1[ex])
                out[m] = out[m] + score32[m, j:j + 1] * (h @ w2[ex].t() + b2[ex])
    return out


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("num_expert,top_k,d,h,batch,act", [
    (4, 2, 64, 128, 300, nn.GELU()),
    (8, 3, 128, 256, 1000, nn.ReLU()),
    (2, 1, 256, 512, 64, nn.GELU(approximate="tanh")),
    (4, 2, 64, 128, 257, nn.Sequential(nn.ReLU(), nn.Dropout(0.0))),
])
def test_fused_mlp_forward_backward(dtype, num_expert, top_k, d, h, batch, act):
    from fastmoe_b200 import FMoETransformerMLP
    from fastmoe_b200.ops import fused, native
    torch.manual_seed(42)
    moe = FMoETransformerMLP(num_expert=num_expert, d_model=d, d_hidden=h, top_k=top_k,
                             activation=act).to(DEV).to(dtype)
    with torch.no_grad():
        moe.experts.htoh4.bias.normal_(0, 0.1)
        moe.experts.h4toh.bias.normal_(0, 0.1)
    x = torch.randn(batch, d, device=DEV, dtype=dtype, requires_grad=True)
    assert fused.supports(moe, x, torch.zeros(1, top_k, dtype=torch.long))
    y = moe(x)
    gy = torch.randn_like(y)
    y.backward(gy)
    got = {n: p.grad.float().clone() for n, p in moe.named_parameters()}
    gx = x.grad.float().clone()
    moe.zero_grad()

    # fp32 oracle with the same routing decisions
    x32 = x.detach().float().requires_grad_(True)
    logits = moe.gate.gate(x.detach()).float()
    gw = moe.gate.gate.weight.float().detach().requires_grad_(True)
    gb = moe.gate.gate.bias.float().detach().requires_grad_(True)
    logits32 = x32 @ gw.t() + gb
    _, idx = torch.topk(logits, top_k, dim=-1)
    score32 = torch.softmax(torch.gather(logits32, 1, idx), dim=-1)
    leaves = _fp32_leaves(moe)
    ref = _dense_reference(moe, x32, idx, score32, leaves)
    ref.backward(gy.float())
    w1g, b1g, w2g, b2g = [t.grad for t in leaves]
    tol = 6e-2 if dtype == torch.bfloat16 else 1e-2
    assert torch.allclose(y.float(), ref, atol=tol, rtol=tol), float((y.float() - ref).abs().max())
    assert torch.allclose(gx, x32.grad, atol=tol * 2, rtol=tol)
    scale = batch ** 0.5
    assert torch.allclose(got["experts.htoh4.weight"], w1g, atol=tol * scale, rtol=tol)
    assert torch.allclose(got["experts.h4toh.weight"], w2g, atol=tol * scale, rtol=tol)
    assert torch.allclose(got["experts.htoh4.bias"], b1g, atol=tol * scale, rtol=tol)
    assert torch.allclose(got["experts.h4toh.bias"], b2g, atol=tol * scale, rtol=tol)
    assert torch.allclose(got["gate.gate.weight"], gw.grad, atol=tol * scale, rtol=tol * 2)
    assert native.get().read_status(0) == 0


def test_fused_mlp_with_dropped_slots():
    r"""A gate that drops slots (-1): dropped slots contribute zero and receive zero gradient."""
    from fastmoe_b200 import FMoETransformerMLP
    from fastmoe_b200.gates import GShardGate
    torch.manual_seed(0)
    moe = FMoETransformerMLP(num_expert=4, d_model=64, d_hidden=128, top_k=2,
                             gate=GShardGate).to(DEV).to(torch.bfloat16)
    moe.gate.capacity = (0.3, 0.3)
    x = torch.randn(400, 64, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    seen = {}
    moe.gate_hook = lambda idx, score, _: seen.update(idx=idx.clone(), score=score.detach().clone())
    y = moe(x)
    y.float().sum().backward()
    idx = seen["idx"]
    assert (idx < 0).any()
    ref = _dense_reference(moe, x.detach().float(), idx, seen["score"].float().view(-1, 2))
    assert torch.allclose(y.float(), ref, atol=6e-2, rtol=6e-2)
    assert torch.isfinite(x.grad.float()).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_general_path_on_gpu(dtype):
    r"""Arbitrary experts + FMoELinear in fp32/fp64 on the device (reference-precision kernels)."""
    from fastmoe_b200 import FMoE, FMoETransformerMLP
    from oracle import LinearExpert, moe_bruteforce
    torch.manual_seed(3)
    d = 16
    moe = FMoE(num_expert=4, d_model=d, top_k=2, expert=LinearExpert).to(DEV).to(dtype)
    x = torch.randn(40, d, device=DEV, dtype=dtype, requires_grad=True)
    y = moe(x)
    val, idx = torch.topk(moe.gate.gate(x), 2, dim=-1)
    ref = moe_bruteforce(x, idx, torch.softmax(val, -1), moe.experts)
    assert torch.allclose(y, ref, atol=1e-4)
    y.sum().backward()

    mlp = FMoETransformerMLP(num_expert=4, d_model=16, d_hidden=32, top_k=2).to(DEV).to(dtype)
    x2 = torch.randn(64, 16, device=DEV, dtype=dtype, requires_grad=True)
    y2 = mlp(x2)
    cpu = FMoETransformerMLP(num_expert=4, d_model=16, d_hidden=32, top_k=2).to(dtype)
    cpu.load_state_dict(mlp.state_dict())
    y2c = cpu(x2.detach().cpu())
    assert torch.allclose(y2.cpu(), y2c, atol=1e-4)
    y2.sum().backward()
    assert torch.isfinite(x2.grad).all()


@pytest.mark.parametrize("gate_name", ["NaiveGate", "NoisyGate", "GShardGate", "SwitchGate",
                                       "DCGate", "ZeroGate", "SwipeGate"])
def test_gates_run_on_gpu(gate_name):
    from fastmoe_b200 import FMoETransformerMLP
    from fastmoe_b200 import gates
    torch.manual_seed(1)
    gate = getattr(gates, gate_name)
    top_k = 1 if gate_name == "SwitchGate" else 2
    moe = FMoETransformerMLP(num_expert=4, d_model=64, d_hidden=128, top_k=top_k,
                             gate=gate).to(DEV).to(torch.bfloat16)
    x = torch.randn(128, 64, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = moe(x)
    loss = y.float().pow(2).mean()
    if moe.gate.has_loss:
        loss = loss + moe.gate.get_loss().float().sum()
    loss.backward()
    assert torch.isfinite(y.float()).all() and torch.isfinite(x.grad.float()).all()


def test_smoke_entry():
    import __graft_entry__ as entry
    entry.smoke()
