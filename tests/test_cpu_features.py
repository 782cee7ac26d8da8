r"""CPU tier: API features of the layer (the ground the reference covers with test_mimo.py,
test_zero.py, test_gates.py, plus what it leaves untested: mask values, state-dict layouts,
NoisyGate/ZeroGate/FasterGate, balance metrics, checkpoint resume)."""
import os
import types

import pytest
import torch
import torch.nn as nn

from fastmoe_b200 import FMoE, FMoELinear, FMoETransformerMLP, balance, checkpoint, gates
from fastmoe_b200.transformer import per_expert_state_dict


class _DictGate(gates.NaiveGate):
    def forward(self, inp):
        return super().forward(inp["x"])


class _DictExpert(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.a = nn.Linear(d, d)
        self.b = nn.Linear(2 * d, 3)

    def forward(self, inp, _count=None):
        return {"u": self.a(inp["x"]), "v": self.b(inp["y"])}


def test_pytree_inputs_and_outputs():
    r"""dict inputs with different widths, dict outputs (reference: tests/test_mimo.py)."""
    torch.manual_seed(0)
    d = 6
    moe = FMoE(num_expert=3, d_model=d, top_k=2, gate=_DictGate, expert=_DictExpert)
    x = {"x": torch.randn(11, d), "y": torch.randn(11, 2 * d)}
    out = moe(x)
    assert out["u"].shape == (11, d) and out["v"].shape == (11, 3)
    idx, score = moe.gate(x)
    ref_u = torch.zeros(11, d)
    for t in range(11):
        for j in range(2):
            e = int(idx[t, j])
            ref_u[t] += score[t, j] * moe.experts[e].a(x["x"][t])
    assert torch.allclose(out["u"], ref_u, atol=1e-5)


def test_list_inputs():
    class ListGate(gates.NaiveGate):
        def forward(self, inp):
            return super().forward(inp[0])

    class ListExpert(nn.Module):
        def __init__(self, d):
            super().__init__()
            self.l = nn.Linear(d, d)

        def forward(self, inp, _count=None):
            return [self.l(inp[0]) + inp[1]]

    moe = FMoE(num_expert=2, d_model=4, top_k=1, gate=ListGate, expert=ListExpert)
    out = moe([torch.randn(5, 4), torch.randn(5, 4)])
    assert isinstance(out, list) and out[0].shape == (5, 4)


def test_zero_gate_and_empty_experts():
    r"""ZeroGate sends everything to expert 0: the other experts see zero rows."""
    torch.manual_seed(1)
    moe = FMoETransformerMLP(num_expert=4, d_model=8, d_hidden=16, top_k=2, gate=gates.ZeroGate)
    x = torch.randn(7, 8, requires_grad=True)
    y = moe(x)
    e = moe.experts
    h = nn.GELU()(x @ e.htoh4.weight[0].t() + e.htoh4.bias[0])
    ref = h @ e.h4toh.weight[0].t() + e.h4toh.bias[0]
    assert torch.allclose(y, ref, atol=1e-5)
    y.sum().backward()
    assert float(e.htoh4.weight.grad[1:].abs().max()) == 0.0


def test_mask_and_mask_dict():
    r"""Tokens with mask != 0 skip the experts and receive the constant row of mask_dict."""
    torch.manual_seed(2)
    d = 8
    mask = torch.tensor([0, 1, 0, 2, 0, 0, 1, 0])
    fill = {1: torch.full((d,), 3.0), 2: torch.full((d,), -1.0)}
    moe = FMoETransformerMLP(num_expert=2, d_model=d, d_hidden=16, top_k=2, mask=mask, mask_dict=fill)
    plain = FMoETransformerMLP(num_expert=2, d_model=d, d_hidden=16, top_k=2)
    plain.load_state_dict(moe.state_dict())
    x = torch.randn(8, d)
    y = moe(x)
    ref = plain(x)
    assert torch.allclose(y[mask == 0], ref[mask == 0], atol=1e-5)
    _, score = moe.gate(x)
    for value, row in fill.items():
        sel = mask == value
        assert torch.allclose(y[sel], score[sel].sum(-1, keepdim=True) * row, atol=1e-5)


def test_state_dict_layouts():
    r"""Fused [E, out, in] layout natively; the per-expert ModuleList layout loads and can be emitted."""
    moe = FMoETransformerMLP(num_expert=3, d_model=4, d_hidden=8, top_k=2)
    sd = moe.state_dict()
    assert sd["experts.htoh4.weight"].shape == (3, 8, 4)
    assert sd["experts.h4toh.weight"].shape == (3, 4, 8)
    assert sd["experts.htoh4.bias"].shape == (3, 8)
    assert sd["gate.gate.weight"].shape == (3, 4) and sd["gate.gate.bias"].shape == (3,)
    per = per_expert_state_dict(sd)
    assert per["experts.1.htoh4.weight"].shape == (1, 8, 4)
    other = FMoETransformerMLP(num_expert=3, d_model=4, d_hidden=8, top_k=2)
    other.load_state_dict(per)
    assert torch.equal(other.experts.h4toh.weight, moe.experts.h4toh.weight)
    for name, p in moe.named_parameters():
        assert p.dp_comm == ("gate" if name.startswith("gate") else "none")


def test_fmoe_linear_shapes_and_repr():
    lin = FMoELinear(4, 8, 16, bias=True, rank=3)
    assert lin.weight.shape == (4, 16, 8) and float(lin.bias.abs().max()) == 0.0
    assert "rank=3" in repr(lin)
    out = lin(torch.randn(6, 8), torch.tensor([1, 2, 0, 3]))
    assert out.shape == (6, 16)


@pytest.mark.parametrize("name,topk", [("NoisyGate", 2), ("GShardGate", 2), ("SwitchGate", 1),
                                       ("DCGate", 2), ("NaiveGate", 3), ("SwipeGate", 2)])
def test_gate_contracts(name, topk):
    torch.manual_seed(3)
    gate = getattr(gates, name)(16, 4, 1, topk)
    gate.train()
    x = torch.randn(50, 16)
    idx, score = gate(x)
    assert idx.shape == (50, topk)
    assert score.reshape(50, -1).shape == (50, topk)
    assert int(idx.max()) < 4 and int(idx.min()) >= -1
    if name != "SwipeGate":   # SWIPE balances by construction and leaves no loss
        assert gate.has_loss
        loss = gate.get_loss()
        assert not gate.has_loss and torch.isfinite(loss).all()


def test_gshard_capacity_and_scores():
    r"""Kept experts respect ceil(cap·B)·k/E and scores equal the softmax of the top-2 logits
    (reference: tests/test_gates.py:35-62)."""
    torch.manual_seed(4)
    n, e = 200, 4
    gate = gates.GShardGate(16, e, 1, capacity=(0.4, 0.4), random_routing=False)
    x = torch.randn(n, 16)
    idx, score = gate(x)
    import math
    cap = math.ceil(0.4 * n) * 2 // e
    counts = torch.bincount(idx[idx >= 0], minlength=e)
    assert int(counts.max()) <= cap
    val, _ = torch.topk(gate.gate(x), 2, dim=-1)
    assert torch.allclose(score, torch.softmax(val, -1), atol=1e-6)


def test_switch_capacity():
    torch.manual_seed(5)
    import math
    n, e = 128, 4
    gate = gates.SwitchGate(16, e, 1, capacity=(0.5, 0.5))
    gate.eval()
    idx, score = gate(torch.randn(n, 16))
    counts = torch.bincount(idx[idx >= 0].reshape(-1), minlength=e)
    assert int(counts.max()) <= math.ceil(0.5 * n / e)
    assert (idx < 0).any()


def test_faster_gate_keeps_most_tokens_local():
    r"""At most ceil(B·fraction) first choices leave the node (reference: tests/test_faster_gate.py)."""
    os.environ["FMOE_TOPO_GPUS_PER_NODE"] = "2"
    os.environ["FMOE_TOPO_OUTGOING_FRACTION"] = "0.1"
    try:
        from fastmoe_b200.gates.faster_gate import FasterGate
        torch.manual_seed(6)
        n_exp, world = 2, 4
        gate = FasterGate(16, n_exp, world, node_rank=1)
        x = torch.randn(100, 16)
        idx, score = gate(x)
        assert (idx >= 0).all()
        node_of = idx // (2 * n_exp)
        leaving = (node_of != 1).any(dim=1).sum()
        assert int(leaving) <= 10
        assert torch.allclose(score.sum(-1), torch.ones(100), atol=1e-5)
    finally:
        del os.environ["FMOE_TOPO_GPUS_PER_NODE"]
        del os.environ["FMOE_TOPO_OUTGOING_FRACTION"]


def test_balance_metrics():
    prof = {}
    balance.reset_balance_profile(prof, 2, "gshard")
    assert set(prof) == set(balance.metrics) | {"gshard_loss"}
    idx = torch.tensor([[0, 1], [0, 2], [0, 1], [3, 0]])
    balance.update_balance_profile(prof, idx, None, torch.tensor(0.5), 1, 4, "gshard")
    c = torch.tensor([4.0, 2.0, 1.0, 1.0])
    assert torch.allclose(prof["Lmax-over-Lmean"][1], c.max() / c.mean())
    assert prof["Lmax-over-Lmin"][0] is None and float(prof["gshard_loss"][1]) == 0.5


def test_checkpoint_resume_is_bitwise(tmp_path):
    r"""save → load into a fresh model/optimizer → the next step is bit-identical."""
    def make():
        torch.manual_seed(7)
        m = FMoETransformerMLP(num_expert=2, d_model=8, d_hidden=16, top_k=2)
        return m, torch.optim.Adam(m.parameters(), lr=1e-2)

    def step(m, o, seed):
        torch.manual_seed(seed)
        x = torch.randn(16, 8)
        o.zero_grad()
        m(x).pow(2).mean().backward()
        o.step()

    m1, o1 = make()
    step(m1, o1, 0)
    checkpoint.save(str(tmp_path), 1, m1, o1, extra={"note": "x"})
    step(m1, o1, 1)
    m2, o2 = make()
    loaded, extra = checkpoint.load(str(tmp_path), m2, o2)
    assert loaded == 1 and extra == {"note": "x"}
    step(m2, o2, 1)
    for a, b in zip(m1.parameters(), m2.parameters()):
        assert torch.equal(a, b)
    assert os.path.exists(os.path.join(str(tmp_path), "step_00000001", "experts_rank0000.pt"))


def test_megatron_adapter_single_process():
    r"""fmoefy + patch_forward_step on the Megatron-shaped GPT with the stand-in megatron objects."""
    from fastmoe_b200.megatron import stub
    from fastmoe_b200.models import GPTConfig, GPTModel
    args = types.SimpleNamespace(hidden_size=16, num_layers=2, balance_strategy="gshard",
                                 balance_loss_weight=0.5, init_method_std=0.02, num_experts=None)
    stub.install(args)
    try:
        from fastmoe_b200 import megatron as fm
        cfg = GPTConfig(hidden_size=16, num_layers=2, num_attention_heads=2, ffn_hidden_size=32,
                        vocab_size=50, max_position_embeddings=8)
        model = fm.fmoefy(GPTModel(cfg), fmoe_num_experts=4, distributed_experts=False,
                          hidden_hidden_size=16, top_k=2, megatron_version="v3.0.2")
        assert all(isinstance(l.mlp, fm.MegatronMLP) for l in model.language_model.encoder.layers)
        assert model.language_model.encoder.layers[0].mlp.experts.htoh4.weight.shape == (4, 16, 16)
        assert len(fm.get_balance_profile()["Lmax-over-Lmean"]) == 2
        tokens = torch.randint(0, 50, (2, 8))

        def forward_step(data_iterator, model, input_tensor):
            loss = model(tokens, tokens)
            return loss, {"lm loss": loss.detach()}

        patched = fm.patch_forward_step(forward_step, "v2.2")
        loss, stats = patched(None, model, None)
        assert "gshard_loss" in stats and torch.isfinite(loss)
        loss.backward()
        assert fm.get_balance_profile()["Lmax-over-Lmean"][0] is not None

        def forward_step25(data_iterator, model):
            out = model(tokens, tokens)
            return out, (lambda o: (o, {"lm loss": o.detach()}))

        out, loss_func, bal = fm.patch_forward_step(forward_step25, "v3.0.2")(None, model)
        total, stats = loss_func(out)
        assert "gshard_loss" in stats and float(bal) > 0

        import argparse
        parser = fm.add_fmoe_args(argparse.ArgumentParser())
        ns = parser.parse_args(["--fmoefy", "--num-experts", "8", "--balance-strategy", "switch"])
        assert ns.fmoefy and ns.num_experts == 8 and ns.top_k == 2 and ns.balance_loss_weight == 1
    finally:
        stub.uninstall()


def test_transformer_xl_memory_and_moe():
    from fastmoe_b200.models import MemTransformerLM
    torch.manual_seed(8)
    lm = MemTransformerLM(n_token=40, n_layer=2, n_head=2, d_model=16, d_head=8, d_inner=32,
                          dropout=0.0, tgt_len=6, mem_len=6, moe=True, moe_num_expert=3, moe_top_k=2)
    data = torch.randint(0, 40, (6, 2))
    out = lm(data, data)
    assert out[0].shape == (6, 2) and len(out) == 1 + 3 and out[1].shape == (6, 2, 16)
    out2 = lm(data, data, *out[1:])
    # the second segment attends to the memory: its loss differs from a memory-less pass
    # (slightly: the weights are drawn with a standard deviation of 0.02)
    assert float((out2[0] - out[0]).abs().max()) > 1e-6
    # ... and an adaptive embedding / softmax variant runs the same recurrence
    lm_ad = MemTransformerLM(n_token=40, n_layer=1, n_head=2, d_model=16, d_head=8, d_inner=32,
                             dropout=0.0, tgt_len=6, mem_len=6, cutoffs=(10, 20), div_val=2)
    o = lm_ad(data, data)
    assert o[0].shape == (6, 2) and torch.isfinite(o[0]).all() and lm_ad.crit is not None
    out2[0].mean().backward()
    assert lm.layers[0].pos_ff.experts.htoh4.weight.grad is not None


def test_debug_routing_check_and_nvtx_switch(monkeypatch):
    r"""``FMOE_DEBUG_BOUNDS`` validation accepts a consistent routing table and names what is
    wrong with an inconsistent one; ``FMOE_NVTX`` ranges are inert without CUDA."""
    from fastmoe_b200 import config
    from fastmoe_b200.ops import api
    from fastmoe_b200.utils.profiling import check_routing, fused_range
    idx = torch.tensor([0, 1, 1, -1, 2, 0])
    cnt, rank = api.route(idx, 3)
    offs = torch.cat([torch.zeros(1, dtype=torch.long), cnt.long().cumsum(0)])
    check_routing(idx, rank, cnt, 3, offs, 6)
    with pytest.raises(ValueError, match="out of range"):
        check_routing(torch.tensor([0, 5]), torch.tensor([0, 0]), torch.tensor([1, 0, 0]), 3)
    with pytest.raises(ValueError, match="share a rank"):
        check_routing(idx, torch.tensor([0, 0, 0, -1, 0, 1]), cnt, 3)
    with pytest.raises(ValueError, match="exceed the buffer"):
        check_routing(idx, rank, cnt, 3, offs, 4)
    monkeypatch.setenv("FMOE_NVTX", "1")
    assert config.nvtx_enabled()
    with fused_range("unit-test"):
        pass
    monkeypatch.setenv("FMOE_DEBUG_BOUNDS", "1")
    assert config.debug_bounds()


def test_ep_trace_summary_arithmetic(monkeypatch):
    r"""The phase summary of the in-kernel time stamps: CTAs that never ran are ignored, phases a
    CTA never reached (stamp 0) do not enter the statistics."""
    from fastmoe_b200 import config
    from fastmoe_b200.utils.profiling import summarize_ep_trace
    stamps = torch.tensor([[1000, 3000, 9000, 20000, 1500, 2000, 4000, 5000, 6000, 2],
                           [2000, 2500, 0, 21000, 0, 0, 0, 0, 4000, 1],
                           [1500, 0, 0, 19000, 0, 0, 0, 0, 0, 0],
                           [0, 0, 0, 0, 0, 0, 0, 0, 0, 0]])
    got = summarize_ep_trace(stamps.reshape(-1))
    assert got["ctas"] == 3
    assert got["launch_skew_us"] == pytest.approx(1.0)
    assert got["kernel_us"] == pytest.approx(20.0)
    assert got["first_rows_us"]["max"] == pytest.approx(2.0)
    assert got["sender_us"] == pytest.approx(8.0)
    assert got["rows_wait_us"] == {"median": pytest.approx(4.0), "max": pytest.approx(6.0), "tiles_waited": 3}
    assert got["first_unit_us"] == {"ids_loaded": pytest.approx(0.5), "stores_issued": pytest.approx(1.0),
                                    "fenced": pytest.approx(3.0), "counted": pytest.approx(4.0)}
    assert summarize_ep_trace(torch.zeros(20, dtype=torch.long)) is None
    assert not config.ep_trace()
    monkeypatch.setenv("FMOE_EP_TRACE", "1")
    assert config.ep_trace()


def test_signal_audit_findings(monkeypatch):
    r"""``SymmWorkspace.audit`` on a stand-in workspace (plain CPU tensors): a state at rest is
    ``ok``; a flag ahead of the epoch, a completion counter or a sender block counter that is
    not zero, a lease that was not handed back and a status code are each found."""
    import types
    from fastmoe_b200.ops import native
    from fastmoe_b200.parallel import symm

    class _Native:
        P2P_NUM_CHANNELS, P2P_MAX_PEERS, P2P_CHAN_REDUCE = 4, 16, 3
        status = 0

        def read_status(self, _index):
            return self.status

    fake_native = _Native()
    monkeypatch.setattr(native, "get", lambda: fake_native)
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)

    def workspace():
        ws = types.SimpleNamespace()
        ws.device = types.SimpleNamespace(index=0)
        ws.world = 2
        ws.epoch = torch.tensor([7, 0, 0, 0, 0, 0, 3, 0], dtype=torch.int32)
        signal = torch.zeros(4, 16, dtype=torch.int32)
        signal[0:3, :2] = 7                 # counts / dispatch / return channels at the exchange epoch
        signal[3, :2] = 2 * 3 + 1           # reduction channel: "done" of reduction 3
        ws.signal = signal.view(torch.uint8).reshape(-1)
        gate = torch.zeros(5, 16, dtype=torch.int32)
        gate[:3, :2] = 7
        gate[3, 0] = 6                      # a block that the last exchange did not touch
        ws._buffers = {"gate": (gate.view(torch.uint8).reshape(-1), [], None)}
        ws._item_count = torch.zeros(9, dtype=torch.int32)
        ws._pool = {1 << 20: [("t", "p")]}
        ws._leased_handles = ["h"]
        return ws

    audit = symm.SymmWorkspace.audit
    rest = audit(workspace())
    assert rest["ok"] and rest["flags_ahead_of_epoch"] == 0 and rest["leases_outstanding"] == 0

    ws = workspace()
    ws._buffers["gate"][0].view(torch.int32).view(5, 16)[4, 1] = 8
    assert audit(ws)["flags_ahead_of_epoch"] == 1 and not audit(ws)["ok"]
    ws = workspace()
    ws.signal.view(torch.int32).view(4, 16)[3, 0] = 2 * 3 + 2
    assert audit(ws)["flags_ahead_of_epoch"] == 1
    ws = workspace()
    ws.epoch[4] = 5
    assert audit(ws)["completion_counters"] == [0, 0, 0, 5, 0] and not audit(ws)["ok"]
    ws = workspace()
    ws._item_count[2] = 40
    assert audit(ws)["sender_block_counters_nonzero"] == 1 and not audit(ws)["ok"]
    ws = workspace()
    ws._pool = {1 << 20: []}
    assert audit(ws)["leases_outstanding"] == 1 and not audit(ws)["ok"]
    fake_native.status = 201
    assert audit(workspace())["status"] == 201 and not audit(workspace())["ok"]


def test_async_gradient_allreduce_handle_without_gpu():
    r"""``allreduce_gradients(async_op=True)`` returns a handle on every device; without CUDA the
    reduction has already happened when it returns."""
    import torch.distributed as dist
    from fastmoe_b200 import DistributedGroupedDataParallel
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29611")
        dist.init_process_group("gloo", rank=0, world_size=1)
        created = True
    else:
        created = False
    try:
        layer = FMoETransformerMLP(num_expert=2, d_model=8, d_hidden=16, world_size=1, top_k=2)
        model = DistributedGroupedDataParallel(layer)
        model(torch.randn(5, 8)).sum().backward()
        before = layer.gate.gate.weight.grad.clone()
        handle = model.allreduce_params(async_op=True)
        handle.wait()
        assert torch.allclose(layer.gate.gate.weight.grad, before)
    finally:
        if created:
            dist.destroy_process_group()


def test_native_smart_schedule_planner_matches_python():
    r"""The C++ chunk planner of the group-wise exchange and its Python restatement agree."""
    from fastmoe_b200.fastermoe import schedule
    from fastmoe_b200.ops import native
    if not native.available():
        pytest.skip("native extension not built")
    gen = torch.Generator().manual_seed(5)
    for world, n_exp, gsz in ((4, 2, 2), (8, 3, 4), (4, 1, 1), (2, 2, 2), (6, 2, 3)):
        for me in range(world):
            tot = world * n_exp
            lec = torch.randint(0, 7, (tot,), generator=gen)
            gec = torch.randint(0, 7, (tot,), generator=gen)
            stored = torch.rand(tot, generator=gen) < 0.3
            got = schedule.plan_steps(lec, gec, stored, n_exp, world, me, gsz)
            want = schedule._plan_steps_python(lec.tolist(), gec.tolist(), stored.tolist(), n_exp,
                                               world, me, gsz)
            assert got[0] == want[0] and got[1] == want[1] and got[2] == want[2]
            assert got[3] == want[3], (world, n_exp, gsz, me)


def test_scatter_gather_rows_and_gradients():
    r"""``MOEScatter`` puts row ``pos // k`` of the input at every kept slot (dropped slots, id -1,
    are skipped), ``MOEGather`` is its transpose, and both pass a numerical gradient check."""
    from fastmoe_b200.functions import MOEGather, MOEScatter, prepare_forward
    torch.manual_seed(12)
    k, n_tok, n_exp, d = 2, 6, 3, 4
    gate = torch.randint(0, n_exp, (n_tok, k))
    gate[1, 0] = -1
    gate[4, 1] = -1
    pos, lec, gec, _cnt, fwd = prepare_forward(gate, n_exp, 1)
    assert fwd == n_tok * k - 2 and pos.numel() == fwd
    x = torch.randn(n_tok, d, dtype=torch.float64, requires_grad=True)
    token_of_slot = torch.div(pos, k, rounding_mode="floor")
    rows = MOEScatter.apply(x, token_of_slot, lec, gec, fwd, 1)
    assert torch.equal(rows, x.detach()[token_of_slot])
    # rows arrive grouped by ascending expert id
    experts_of_rows = gate.reshape(-1)[pos]
    assert torch.equal(experts_of_rows, experts_of_rows.sort().values)
    assert torch.autograd.gradcheck(
        lambda t: MOEScatter.apply(t, token_of_slot, lec, gec, fwd, 1), (x,))
    y = torch.randn(fwd, d, dtype=torch.float64, requires_grad=True)
    back = MOEGather.apply(y, pos, lec, gec, n_tok * k, 1)
    assert back.shape == (n_tok * k, d)
    assert torch.equal(back[pos], y.detach()) and float(back[1 * k + 0].abs().sum()) == 0.0
    assert torch.autograd.gradcheck(
        lambda t: MOEGather.apply(t, pos, lec, gec, n_tok * k, 1), (y,))
