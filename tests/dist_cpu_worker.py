r"""Worker of the CPU multi-process tests (gloo): one process per emulated rank."""
import os
import sys
import time

import torch
import torch.distributed as dist
import torch.nn as nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from fastmoe_b200 import DistributedGroupedDataParallel, FMoETransformerMLP  # noqa: E402
from fastmoe_b200 import gates  # noqa: E402
from oracle import moe_mlp_bruteforce  # noqa: E402


def _gather(t):
    parts = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, t.contiguous())
    return parts


def case_ep_matches_bruteforce():
    r"""Expert-parallel layer (general path) == brute force over the gathered experts."""
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(7)  # same gate on every rank
    moe = FMoETransformerMLP(num_expert=2, d_model=8, d_hidden=16, world_size=world, top_k=2)
    torch.manual_seed(100 + rank)  # different experts and data per rank
    for p in moe.experts.parameters():
        nn.init.normal_(p, std=0.3)
    x = torch.randn(10 + rank, 8, requires_grad=True)
    y = moe(x)
    y.sum().backward()

    e = moe.experts
    w1 = torch.cat(_gather(e.htoh4.weight.detach()))
    b1 = torch.cat(_gather(e.htoh4.bias.detach()))
    w2 = torch.cat(_gather(e.h4toh.weight.detach()))
    b2 = torch.cat(_gather(e.h4toh.bias.detach()))
    x2 = x.detach().clone().requires_grad_(True)
    val, idx = torch.topk(moe.gate.gate(x2), 2, dim=-1)
    ref = moe_mlp_bruteforce(x2, idx, torch.softmax(val, -1), w1, b1, w2, b2, nn.GELU())
    ref.sum().backward()
    assert torch.allclose(y, ref, atol=1e-5), (y - ref).abs().max()
    assert torch.allclose(x.grad, x2.grad, atol=1e-5)


def case_capacity_gates():
    r"""Switch / DC / GShard gates respect their capacities across ranks."""
    world = dist.get_world_size()
    torch.manual_seed(3)
    n_tok, n_exp = 64, 2
    for name, topk in (("SwitchGate", 1), ("DCGate", 2), ("GShardGate", 2)):
        gate = getattr(gates, name)(8, n_exp, world, topk, capacity=(0.5, 0.5))
        gate.train()
        x = torch.randn(n_tok, 8)
        idx, score = gate(x)
        assert idx.shape == (n_tok, topk)
        counts = torch.bincount(idx[idx >= 0].reshape(-1), minlength=n_exp * world)
        tot = counts.clone()
        dist.all_reduce(tot)
        if name == "SwitchGate":
            cap = -(-int(0.5 * n_tok) // n_exp) if False else int(torch.ceil(torch.tensor(0.5 * n_tok / n_exp)))
            assert int(tot.max()) <= cap, (name, tot, cap)
        elif name == "DCGate":
            assert int(tot.max()) <= int(0.5 * n_tok + 0.999), (name, tot)
        else:
            cap = int(0.5 * n_tok + 0.999) * 2 // (n_exp * world)
            assert int(counts.max()) <= cap, (name, counts, cap)
        assert gate.has_loss


def case_swipe_gate():
    world = dist.get_world_size()
    from fastmoe_b200.functions import ensure_comm
    ensure_comm(torch.zeros(1), None)
    torch.manual_seed(11 + dist.get_rank())
    gate = gates.SwipeGate(8, 2, world, 2)
    gate.train()
    x = torch.randn(32, 8)
    idx, score = gate(x)
    assert idx.shape == (32, 2) and (idx >= 0).all() and (idx < 2 * world).all()
    # no worker receives more than batch * top_k tokens
    worker = torch.div(idx.reshape(-1), 2, rounding_mode="floor")
    load = torch.bincount(worker, minlength=world)
    dist.all_reduce(load)
    assert int(load.max()) <= 32 * 2, load
    assert torch.allclose(score.sum(-1), torch.ones(32), atol=1e-5)


def case_grouped_ddp():
    r"""Gate grads are averaged over the world, expert grads ('none') are left alone."""
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(5 + rank)
    moe = FMoETransformerMLP(num_expert=2, d_model=8, d_hidden=16, world_size=world, top_k=2)
    model = DistributedGroupedDataParallel(moe)
    gate_w = _gather(moe.gate.gate.weight.detach())
    assert all(torch.equal(gate_w[0], g) for g in gate_w), "gate not synchronised at construction"
    x = torch.randn(12, 8)
    model(x).pow(2).sum().backward()
    local_gate = moe.gate.gate.weight.grad.clone()
    local_exp = moe.experts.htoh4.weight.grad.clone()
    model.allreduce_params()
    expect = torch.stack(_gather(local_gate)).mean(0)
    assert torch.allclose(moe.gate.gate.weight.grad, expect, atol=1e-6)
    assert torch.equal(moe.experts.htoh4.weight.grad, local_exp)


def case_hybrid_dp_ep():
    r"""Hybrid data x expert parallelism on 4 ranks: ranks {0,1} and {2,3} are two expert-parallel
    groups, the experts of rank r and rank r+2 are replicas (tag 'dp', reduced over {r, r+2}),
    gates are reduced over all ranks.  After the reduction the replicas hold identical gradients
    and they equal the average of the two groups' own gradients."""
    rank, world = dist.get_rank(), dist.get_world_size()
    assert world == 4
    ep_groups = [dist.new_group([0, 1]), dist.new_group([2, 3])]
    dp_groups = [dist.new_group([0, 2]), dist.new_group([1, 3])]
    ep_group, dp_group = ep_groups[rank // 2], dp_groups[rank % 2]
    torch.manual_seed(70 + rank % 2)              # replicas start from the same experts
    moe = FMoETransformerMLP(num_expert=2, d_model=8, d_hidden=16, world_size=2, moe_group=ep_group,
                             top_k=2, expert_dp_comm="dp")
    model = DistributedGroupedDataParallel(moe, dp_group=dp_group, moe_group=ep_group,
                                           gate_group=dist.group.WORLD)
    # construction synchronised every tag inside its group
    rep = [torch.empty_like(moe.experts.htoh4.weight) for _ in range(2)]
    dist.all_gather(rep, moe.experts.htoh4.weight.detach().contiguous(), group=dp_group)
    assert torch.equal(rep[0], rep[1])
    gates_all = _gather(moe.gate.gate.weight.detach())
    assert all(torch.equal(gates_all[0], g) for g in gates_all)
    for p in moe.experts.parameters():
        assert p.dp_comm == "dp"
    torch.manual_seed(90 + rank)                  # different data everywhere
    model(torch.randn(10, 8)).pow(2).sum().backward()
    own_expert = moe.experts.htoh4.weight.grad.clone()
    own_gate = moe.gate.gate.weight.grad.clone()
    model.allreduce_params()
    pair = [torch.empty_like(own_expert) for _ in range(2)]
    dist.all_gather(pair, own_expert, group=dp_group)
    assert torch.allclose(moe.experts.htoh4.weight.grad, (pair[0] + pair[1]) / 2, atol=1e-6)
    assert torch.allclose(moe.gate.gate.weight.grad, torch.stack(_gather(own_gate)).mean(0), atol=1e-6)


def case_slice_group():
    r"""slice_group: ranks share the input, each routes its slice, outputs are all-gathered."""
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(9)
    moe = FMoETransformerMLP(num_expert=2, d_model=8, d_hidden=16, world_size=1, top_k=2,
                             slice_group=dist.group.WORLD)
    x = torch.randn(4 * world, 8, requires_grad=True)
    y = moe(x)
    assert y.shape == x.shape
    ref_layer = FMoETransformerMLP(num_expert=2, d_model=8, d_hidden=16, world_size=1, top_k=2)
    ref_layer.load_state_dict(moe.state_dict())
    ref = ref_layer(x.detach())
    assert torch.allclose(y, ref, atol=1e-5)
    y.sum().backward()
    assert x.grad.shape == x.shape
    # Remainder rows (batch not divisible by the group size) are not routed, as in the
    # reference: Slice keeps B // W rows per rank and its backward leaves the tail at zero.
    from fastmoe_b200.functions import AllGather, Slice
    full = torch.arange((4 * world + 1) * 3, dtype=torch.float32).view(4 * world + 1, 3).requires_grad_(True)
    part = Slice.apply(full, rank, world, dist.group.WORLD)
    assert part.shape[0] == 4 and torch.equal(part, full.detach()[4 * rank:4 * rank + 4])
    gathered = AllGather.apply(part * 2.0, rank, world, dist.group.WORLD)
    assert torch.equal(gathered, 2.0 * full.detach()[:4 * world])
    gathered.sum().backward()
    assert torch.equal(full.grad[:4 * world], torch.full((4 * world, 3), 2.0))
    assert float(full.grad[4 * world:].abs().sum()) == 0.0


def case_pipeline_hybrid():
    r"""Pipeline x expert parallelism (2 stages x 2 ranks): the 1F1B runner with MoE stages gives
    the loss and the gradients of the same model run in one process; expert gradients are summed
    over the data-parallel chains, shared ones averaged; the balance loss of every stage is
    back-propagated with weight / n_stages."""
    from fastmoe_b200.parallel.pipeline import PipelineRunner, build_stage_groups
    rank, world = dist.get_rank(), dist.get_world_size()
    n_stages, n_micro, tokens, d, h, n_exp, blocks_per_stage = 2, 3, 6, 8, 16, 2, 2
    stage, group, prev_rank, next_rank = build_stage_groups(n_stages)
    ssize = world // n_stages
    chain = rank % ssize

    class Block(nn.Module):
        def __init__(self, num_expert, world_size, moe_group, gate):
            super().__init__()
            self.lin = nn.Linear(d, d)
            self.moe = FMoETransformerMLP(num_expert=num_expert, d_model=d, d_hidden=h, top_k=2,
                                          world_size=world_size, moe_group=moe_group, gate=gate)

        def forward(self, x):
            return x + self.moe(torch.tanh(self.lin(x)))

    def data(j):
        gen = torch.Generator().manual_seed(300 + j)
        xs = [torch.randn(tokens, d, generator=gen) for _ in range(n_micro)]
        ts = [torch.randn(tokens, d, generator=gen) for _ in range(n_micro)]
        return xs, ts

    def mse(out, target):
        return (out - target).pow(2).mean()

    gate_grads = {}
    for gate_cls, weight in ((gates.NaiveGate, 0.0), (gates.GShardGate, 0.0), (gates.GShardGate, 0.5),
                             (gates.GShardGate, 1.0)):
        torch.manual_seed(17)
        full = nn.Sequential(*[Block(n_exp * ssize, 1, None, gate_cls)
                               for _ in range(n_stages * blocks_per_stage)])
        mine = nn.Sequential(*[Block(n_exp, ssize, group, gate_cls) for _ in range(blocks_per_stage)])
        refs = list(full)[stage * blocks_per_stage:(stage + 1) * blocks_per_stage]
        lo, hi = chain * n_exp, (chain + 1) * n_exp
        for b, ref in zip(mine, refs):
            b.lin.load_state_dict(ref.lin.state_dict())
            b.moe.gate.load_state_dict(ref.moe.gate.state_dict())
            with torch.no_grad():
                for name in ("htoh4", "h4toh"):
                    getattr(b.moe.experts, name).weight.copy_(getattr(ref.moe.experts, name).weight[lo:hi])
                    getattr(b.moe.experts, name).bias.copy_(getattr(ref.moe.experts, name).bias[lo:hi])
        model = DistributedGroupedDataParallel(mine, dp_group=group, gate_group=group, moe_group=group,
                                               need_sync=False)
        xs, ts = data(chain)
        runner = PipelineRunner(mine, stage, n_stages, prev_rank, next_rank, (tokens, d), torch.float32,
                                loss_fn=mse, balance_weight=weight)
        torch.manual_seed(23)          # GShard's random second-expert routing: same draws in every run
        loss = runner.run(micro_batches=xs if stage == 0 else None,
                          targets=ts if stage == n_stages - 1 else None, n_micro=n_micro)
        model.allreduce_params()

        if gate_cls is gates.NaiveGate:
            # single-process reference over the data of both chains
            total = 0.0
            for j in range(ssize):
                xj, tj = data(j)
                for x, t in zip(xj, tj):
                    total = total + mse(full(x), t) / (n_micro * ssize)
            total.backward()
            if stage == n_stages - 1:
                mean = loss.clone()
                dist.all_reduce(mean, group=group)
                assert torch.allclose(mean / ssize, total.detach(), atol=1e-5), (mean / ssize, total)
            for b, ref in zip(mine, refs):
                assert torch.allclose(b.lin.weight.grad, ref.lin.weight.grad, atol=1e-5)
                assert torch.allclose(b.moe.gate.gate.weight.grad, ref.moe.gate.gate.weight.grad, atol=1e-5)
                want = ref.moe.experts.htoh4.weight.grad[lo:hi] * ssize
                assert torch.allclose(b.moe.experts.htoh4.weight.grad, want, atol=1e-5)
        else:
            gate_grads[weight] = torch.cat([b.moe.gate.gate.weight.grad.reshape(-1) for b in mine]).clone()
    # Every stage back-propagates weight / n_stages times its own balance loss: the gate
    # gradients are affine in the weight, and the balance term is not zero on any stage.
    g0, g1, g2 = gate_grads[0.0], gate_grads[0.5], gate_grads[1.0]
    assert torch.allclose(g2 - g1, g1 - g0, atol=1e-5), float(((g2 - g1) - (g1 - g0)).abs().max())
    assert float((g1 - g0).abs().max()) > 1e-6, "the balance loss did not reach the gates of stage %d" % stage


def case_smart_schedule():
    r"""Smart schedule (all group sizes, with and without shadow experts) == general path."""
    from fastmoe_b200.fastermoe import schedule
    from fastmoe_b200.functions import ensure_comm
    from fastmoe_b200.layers import _fmoe_general_global_forward as naive_forward
    from oracle import LinearExpert
    from fastmoe_b200 import FMoE
    rank, world = dist.get_rank(), dist.get_world_size()
    ensure_comm(torch.zeros(1), None)
    for fused_experts in (False, True):
        for group_size in (1, 2, 4):
            for shadow in (False, True):
                os.environ["FMOE_FASTER_GROUP_SIZE"] = str(group_size)
                torch.manual_seed(21 + rank)
                if fused_experts:
                    layer = FMoETransformerMLP(num_expert=2, d_model=8, d_hidden=16, world_size=world, top_k=2)
                else:
                    layer = FMoE(num_expert=2, d_model=8, world_size=world, top_k=2, expert=LinearExpert)
                x = torch.randn(9 + rank, 8)
                idx = torch.randint(0, 2 * world, (x.shape[0], 2))
                torch.manual_seed(77)
                stored = torch.rand(2 * world) < 0.4 if shadow else torch.zeros(2 * world, dtype=torch.bool)

                xa = x.clone().requires_grad_(True)
                ya = naive_forward(xa, idx, layer.expert_fn, 2, world)
                ya.pow(2).sum().backward()
                ga = [p.grad.clone() for p in layer.experts.parameters()]
                layer.zero_grad()

                xb = x.clone().requires_grad_(True)
                yb = schedule._fmoe_general_global_forward(
                    xb, idx, layer.expert_fn_single, 2, world, experts=layer.experts, stored_models=stored)
                yb.pow(2).sum().backward()
                gb = [p.grad.clone() for p in layer.experts.parameters()]
                assert torch.allclose(ya, yb, atol=1e-5), (group_size, shadow, (ya - yb).abs().max())
                assert torch.allclose(xa.grad, xb.grad, atol=1e-5)
                for a, b in zip(ga, gb):
                    assert torch.allclose(a, b, atol=1e-4), (group_size, shadow, (a - b).abs().max())


class _CallbackMoEForward(torch.autograd.Function):
    r"""The calling sequence of the reference's ``MoEForward`` (fmoe/fastermoe/schedule.py:15-114)
    around ``fmoe_cuda.smart_sch_forward`` / ``smart_sch_backward`` / ``reduce_grad``."""

    @staticmethod
    def forward(ctx, expert_fn, experts, inp, pos_s, pos_g, lec, gec, stored, fwd_batch, out_batch,
                num_expert, world):
        import fmoe_cuda
        from fastmoe_b200.fastermoe import expert_utils
        from fastmoe_b200.functions import _local_gather, _local_scatter
        local_in = _local_scatter(inp, pos_s)
        ctx.gibs, ctx.gobs = {}, {}

        def run(x, y, expert_idx, store_idx):
            x = x.detach().requires_grad_(True)
            keep = lambda t: t  # noqa: E731
            # parameters are overwritten in place when a shadow is stashed and restored: the
            # identity hooks keep autograd's version check out of the way, as in the reference
            with torch.enable_grad(), torch.autograd.graph.saved_tensors_hooks(keep, keep):
                y0 = expert_fn(x, torch.tensor([x.shape[0]], dtype=torch.int64), expert_idx)
            ctx.gibs[store_idx], ctx.gobs[store_idx] = x, y0
            y.copy_(y0.detach())

        ctx.experts = experts
        ctx.expert_size = expert_utils.get_expert_param_size(experts, 0)
        ctx.shadows = {}

        def stash(params, store_idx, expert_idx):
            expert_utils.stash_expert_params(experts, params, expert_idx)
            ctx.shadows[store_idx] = params

        out_buf, gib = fmoe_cuda.smart_sch_forward(
            local_in, lec, gec, stored, fwd_batch, ctx.expert_size, world, run,
            lambda out, idx: expert_utils.get_expert_params(experts, out, idx), stash,
            lambda idx: expert_utils.pop_expert_params(experts, idx))
        ctx.args = fwd_batch, inp.shape[0], num_expert, world
        ctx.save_for_backward(pos_s, pos_g, lec, gec, stored, gib, local_in)
        return _local_gather(out_buf, pos_g, out_batch, maybe_overlap=False)

    @staticmethod
    def backward(ctx, grad_out):
        import fmoe_cuda
        from fastmoe_b200.fastermoe import expert_utils
        from fastmoe_b200.functions import _local_gather, _local_scatter
        pos_s, pos_g, lec, gec, stored, _gib, _lin = ctx.saved_tensors
        fwd_batch, inp_batch, _num_expert, world = ctx.args
        experts = ctx.experts

        def back(grad_y, grad_x, expert_idx, store_idx):
            y, x = ctx.gobs[store_idx], ctx.gibs[store_idx]
            torch.autograd.backward([y], [grad_y])
            grad_x.copy_(x.grad if x.grad is not None else torch.zeros_like(x))

        def collect(store_idx, root, expert_idx):
            grad = ctx.shadows[store_idx]
            expert_utils.collect_expert_grads(experts, grad, expert_idx)
            fmoe_cuda.reduce_grad(grad, root, ctx.expert_size)

        grad_buf = _local_scatter(grad_out.contiguous(), pos_g)
        grad_in_buf = fmoe_cuda.smart_sch_backward(
            grad_buf, lec, gec, stored, pos_s.shape[0], fwd_batch, world, back,
            lambda store_idx, idx: expert_utils.stash_expert_params(experts, ctx.shadows[store_idx], idx),
            lambda idx: expert_utils.pop_expert_params(experts, idx), collect,
            lambda store_idx, idx: expert_utils.set_grads(experts, ctx.shadows[store_idx], idx))
        grad_in = _local_gather(grad_in_buf, pos_s, inp_batch)
        return (None, None, grad_in) + (None,) * 9


def case_smart_sch_entry_points():
    r"""``fmoe_cuda.smart_sch_forward`` / ``smart_sch_backward`` / ``reduce_grad`` driven with the
    reference's callbacks (per-expert modules, parameters stashed into expert 0 for shadows)
    == the general path."""
    from fastmoe_b200 import FMoE
    from fastmoe_b200.functions import ensure_comm, prepare_forward
    from fastmoe_b200.layers import _fmoe_general_global_forward as naive_forward
    from oracle import LinearExpert
    rank, world = dist.get_rank(), dist.get_world_size()
    ensure_comm(torch.zeros(1), None)
    for group_size in (1, 2):
        for shadow in (False, True):
            os.environ["FMOE_FASTER_GROUP_SIZE"] = str(group_size)
            torch.manual_seed(31 + rank)
            layer = FMoE(num_expert=2, d_model=8, world_size=world, top_k=2, expert=LinearExpert)
            x = torch.randn(11 + rank, 8)
            idx = torch.randint(0, 2 * world, (x.shape[0], 2))
            torch.manual_seed(78)
            stored = torch.rand(2 * world) < 0.4 if shadow else torch.zeros(2 * world, dtype=torch.bool)

            xa = x.clone().requires_grad_(True)
            ya = naive_forward(xa, idx, layer.expert_fn, 2, world)
            ya.pow(2).sum().backward()
            ga = [p.grad.clone() for p in layer.experts.parameters()]
            layer.zero_grad()

            xb = x.clone().requires_grad_(True)
            pos, lec, gec, _fec, fwd_batch = prepare_forward(idx, 2, world)
            yb = _CallbackMoEForward.apply(
                layer.expert_fn_single, layer.experts, xb, torch.div(pos, 2, rounding_mode="floor"), pos,
                lec, gec, stored, fwd_batch, x.shape[0] * 2, 2, world)
            yb.pow(2).sum().backward()
            gb = [torch.zeros_like(p) if p.grad is None else p.grad.clone() for p in layer.experts.parameters()]
            assert torch.allclose(ya, yb, atol=1e-5), (group_size, shadow, float((ya - yb).abs().max()))
            assert torch.allclose(xa.grad, xb.grad, atol=1e-5)
            for a, b in zip(ga, gb):
                assert torch.allclose(a, b, atol=1e-4), (group_size, shadow, float((a - b).abs().max()))


def case_shadow_policy():
    r"""The policy shadows the overloaded expert and nothing when the load is flat."""
    from fastmoe_b200.fastermoe.shadow_policy import shadow_plan
    flat = shadow_plan([100] * 8, 1024, 2, 900e9, 1.3e15, 2)
    assert not any(flat)
    skew = shadow_plan([100000, 10, 10, 10, 10, 10, 10, 10], 1024, 2, 900e9, 1.3e15, 2)
    assert skew[0] and not any(skew[1:])


def case_tensor_parallel():
    r"""Megatron tensor parallelism of the experts: every rank of the tensor-parallel group holds a
    slice of each expert's hidden dimension, the partial outputs are summed
    (``reduce_from_tensor_model_parallel_region``); together they equal one layer whose expert
    weights are the concatenation of the slices (and whose output bias is the sum of the ranks'
    biases, a property of the reference's layout)."""
    import types
    from fastmoe_b200.megatron import stub
    from fastmoe_b200.megatron.layers import MegatronMLP
    rank, world = dist.get_rank(), dist.get_world_size()
    d, hidden_per_rank, n_exp = 8, 6, 3
    args = types.SimpleNamespace(hidden_size=d, num_layers=2, balance_strategy="naive", top_k=2,
                                 init_method_std=0.05, fmoe_num_experts=n_exp, distributed_experts=False,
                                 hidden_hidden_size=hidden_per_rank, tensor_model_parallel_size=world)
    stub.install(args, tensor_parallel_group=dist.group.WORLD)
    import numpy as np
    torch.manual_seed(31)          # same gate on every rank
    np.random.seed(40 + rank)      # different expert slices per rank
    mlp = MegatronMLP(args, 0)
    for p in mlp.experts.parameters():
        with torch.no_grad():
            p.add_(0.01 * (rank + 1))          # also give the biases rank-dependent values
    x = torch.randn(11, d, generator=torch.Generator().manual_seed(5), requires_grad=True)
    out, bias = mlp(x)
    assert bias.shape == (d,) and float(bias.abs().sum()) == 0.0
    out.pow(2).sum().backward()

    full = FMoETransformerMLP(num_expert=n_exp, d_model=d, d_hidden=hidden_per_rank * world, top_k=2)
    full.gate.load_state_dict(mlp.gate.state_dict())
    w1 = torch.cat(_gather(mlp.experts.htoh4.weight.detach()), dim=1)     # [E, world*h, d]
    b1 = torch.cat(_gather(mlp.experts.htoh4.bias.detach()), dim=1)
    w2 = torch.cat(_gather(mlp.experts.h4toh.weight.detach()), dim=2)     # [E, d, world*h]
    b2 = torch.stack(_gather(mlp.experts.h4toh.bias.detach())).sum(0)
    with torch.no_grad():
        full.experts.htoh4.weight.copy_(w1)
        full.experts.htoh4.bias.copy_(b1)
        full.experts.h4toh.weight.copy_(w2)
        full.experts.h4toh.bias.copy_(b2)
    xr = x.detach().clone().requires_grad_(True)
    ref = full(xr)
    assert torch.allclose(out, ref, atol=1e-5), float((out - ref).abs().max())
    ref.pow(2).sum().backward()
    lo, hi = rank * hidden_per_rank, (rank + 1) * hidden_per_rank
    assert torch.allclose(mlp.experts.htoh4.weight.grad, full.experts.htoh4.weight.grad[:, lo:hi], atol=1e-4)
    assert torch.allclose(mlp.experts.h4toh.weight.grad, full.experts.h4toh.weight.grad[:, :, lo:hi], atol=1e-4)
    stub.uninstall()


def case_megatron_checkpoint():
    r"""Megatron adapter under expert parallelism: fmoefy, grouped DDP with a gate group, and
    sharded save / load (rank 0 full file, other ranks expert shards) giving identical models."""
    import types
    from fastmoe_b200.megatron import stub
    from fastmoe_b200.models import GPTConfig, GPTModel
    rank, world = dist.get_rank(), dist.get_world_size()
    save_dir = os.environ["FMOE_TEST_TMP"]
    args = types.SimpleNamespace(hidden_size=16, num_layers=2, balance_strategy="naive",
                                 init_method_std=0.02, save=save_dir, load=save_dir)
    stub.install(args)
    from fastmoe_b200 import megatron as fm
    cfg = GPTConfig(hidden_size=16, num_layers=2, num_attention_heads=2, ffn_hidden_size=32,
                    vocab_size=50, max_position_embeddings=8)

    def build():
        torch.manual_seed(3)
        import numpy as np
        np.random.seed(5)
        model = fm.fmoefy(GPTModel(cfg), fmoe_num_experts=2, distributed_experts=True,
                          hidden_hidden_size=16, top_k=2, megatron_version="v3.0.2")
        return model, fm.DistributedDataParallel(model)

    model, ddp = build()
    mlp = model.language_model.encoder.layers[0].mlp
    assert mlp.world_size == world and mlp.experts.htoh4.weight.dp_comm == "none"
    # experts differ per rank, dense parameters are synchronised
    w = _gather(mlp.experts.htoh4.weight.detach())
    assert not torch.equal(w[0], w[1])
    q = _gather(model.language_model.encoder.layers[0].self_attention.dense.weight.detach())
    assert torch.equal(q[0], q[1])

    opt = torch.optim.Adam(model.parameters(), lr=1e-2)
    tokens = torch.randint(0, 50, (2, 8))
    loss = ddp(tokens, tokens)
    loss.backward()
    ddp.allreduce_params()
    opt.step()
    wrapper = types.SimpleNamespace(optimizer=opt, state_dict=opt.state_dict,
                                    load_state_dict=opt.load_state_dict)
    fm.save_checkpoint(7, ddp, wrapper, None)
    name = "mp_rank_00" if rank == 0 else "mp_rank_00_dp_rank_{:04d}".format(rank)
    path = os.path.join(save_dir, "iter_0000007", name, "model_optim_rng.pt")
    assert os.path.exists(path), path
    if rank > 0:
        shard = torch.load(path, weights_only=False)
        keys = []

        def walk(d, prefix=""):
            for k, v in d.items():
                walk(v, prefix + k + ".") if isinstance(v, dict) else keys.append(prefix + k)

        walk(shard["model"])
        assert keys and all("experts" in k for k in keys), keys

    model2, ddp2 = build()
    for p in model2.parameters():
        torch.nn.init.zeros_(p)
    opt2 = torch.optim.Adam(model2.parameters(), lr=1e-2)
    wrapper2 = types.SimpleNamespace(optimizer=opt2, state_dict=opt2.state_dict,
                                     load_state_dict=opt2.load_state_dict)
    it = fm.load_checkpoint(ddp2, wrapper2, None)
    assert it == 7
    for (n1, p1), (n2, p2) in zip(model.named_parameters(), model2.named_parameters()):
        assert torch.equal(p1, p2), n1
    stub.uninstall()


def case_generic_checkpoint():
    r"""fastmoe_b200.checkpoint under expert parallelism: every rank gets its own experts back."""
    from fastmoe_b200 import checkpoint
    rank, world = dist.get_rank(), dist.get_world_size()
    save_dir = os.environ["FMOE_TEST_TMP"]
    torch.manual_seed(40 + rank)
    moe = FMoETransformerMLP(num_expert=2, d_model=8, d_hidden=16, world_size=world, top_k=2)
    model = DistributedGroupedDataParallel(moe)
    opt = torch.optim.Adam(moe.parameters(), lr=1e-2)
    model(torch.randn(6, 8)).pow(2).mean().backward()
    model.allreduce_params()
    opt.step()
    checkpoint.save(save_dir, 3, moe, opt)
    torch.manual_seed(999)
    fresh = FMoETransformerMLP(num_expert=2, d_model=8, d_hidden=16, world_size=world, top_k=2)
    opt2 = torch.optim.Adam(fresh.parameters(), lr=1e-2)
    step, _ = checkpoint.load(save_dir, fresh, opt2)
    assert step == 3
    for a, b in zip(moe.parameters(), fresh.parameters()):
        assert torch.equal(a, b)
    assert torch.equal(opt.state[moe.experts.htoh4.weight]["exp_avg"],
                       opt2.state[fresh.experts.htoh4.weight]["exp_avg"])


def case_rank_failure():
    r"""A rank that raises before a collective: the others get an error from the bounded
    process-group timeout instead of hanging."""
    rank = dist.get_rank()
    if rank == 1:
        raise SystemExit(3)
    t = torch.ones(1)
    try:
        dist.all_reduce(t)
    except Exception:  # pylint: disable=broad-except
        raise SystemExit(0)
    raise SystemExit(4)


if __name__ == "__main__":
    case = sys.argv[1]
    from datetime import timedelta
    timeout = timedelta(seconds=8 if case == "rank_failure" else 120)
    dist.init_process_group("gloo", timeout=timeout)
    globals()["case_" + case]()
    if case != "rank_failure":
        dist.barrier()
        # Leave without running the process-group and interpreter destructors: with the gloo
        # backend a rank whose peers have already closed their sockets occasionally aborts in
        # a background thread during teardown, after the case itself has passed.
        sys.stdout.flush()
        sys.stderr.flush()
        time.sleep(0.2)
        os._exit(0)
