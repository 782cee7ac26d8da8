r"""Worker of the multi-GPU tests: one process per GPU (NCCL for the comparison path, the
peer-to-peer kernels for the fused path).  No test here faults, traps or hangs a GPU: the
failure case lets a bounded device wait run out and reads the status word."""
import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from fastmoe_b200 import DistributedGroupedDataParallel, FMoETransformerMLP  # noqa: E402
from fastmoe_b200.ops import native  # noqa: E402
from fastmoe_b200.parallel import symm  # noqa: E402


def _dev():
    return torch.device("cuda", int(os.environ["LOCAL_RANK"]))


def _make_layer(world, rank, num_expert=2, d=256, h=512, top_k=2, dtype=torch.bfloat16,
                activation=None):
    torch.manual_seed(7)
    layer = FMoETransformerMLP(num_expert=num_expert, d_model=d, d_hidden=h, world_size=world,
                               top_k=top_k, activation=activation or nn.GELU())
    torch.manual_seed(100 + rank)
    for p in layer.experts.parameters():
        nn.init.normal_(p, std=0.05)
    return layer.to(_dev()).to(dtype)


def _run(layer, x, gy):
    layer.zero_grad()
    xx = x.detach().clone().requires_grad_(True)
    y = layer(xx)
    y.backward(gy)
    grads = {n: p.grad.detach().float().clone() for n, p in layer.named_parameters()}
    return y.detach().float(), xx.grad.detach().float(), grads


def case_fused_vs_general():
    r"""Peer-to-peer fused path == collective-library general path (same kernels for the GEMMs)."""
    rank, world = dist.get_rank(), dist.get_world_size()
    cases = ((2, 2, 512, None), (1, 1, 300, None), (4, 3, 1000, nn.ReLU()),
             (2, 2, 640, nn.Sequential(nn.ReLU(), nn.Dropout(0.0))))
    # the exchange buffers are sized once per group: announce the largest batch of this test
    symm.reserve_tokens(dist.group.WORLD, max(c[2] for c in cases), _dev())
    for num_expert, top_k, n_tok, activation in cases:
        layer = _make_layer(world, rank, num_expert=num_expert, top_k=top_k, activation=activation)
        torch.manual_seed(1000 + rank)
        x = torch.randn(n_tok, 256, device=_dev(), dtype=torch.bfloat16)
        gy = torch.randn(n_tok, 256, device=_dev(), dtype=torch.bfloat16)
        assert symm.fused_available(layer, x), "fused path unavailable"
        y1, gx1, g1 = _run(layer, x, gy)
        os.environ["FMOE_FUSED"] = "0"
        assert not symm.fused_available(layer, x)
        y2, gx2, g2 = _run(layer, x, gy)
        os.environ["FMOE_FUSED"] = "1"
        assert torch.allclose(y1, y2, atol=2e-2, rtol=2e-2), float((y1 - y2).abs().max())
        assert torch.allclose(gx1, gx2, atol=2e-2, rtol=2e-2), float((gx1 - gx2).abs().max())
        for name in g1:
            # bf16 gradients: compare against the magnitude of the tensor
            err = float((g1[name] - g2[name]).abs().max())
            ref = float(g2[name].abs().max())
            assert err <= 0.04 * ref + 1e-3, (name, err, ref)
        assert native.get().read_status(_dev().index) == 0


def _gathered_fp32(layer, world):
    r"""Every rank's expert parameters in one fp32 set, in global expert order (leaf tensors)."""
    e = layer.experts
    out = []
    for t in (e.htoh4.weight, e.htoh4.bias, e.h4toh.weight, e.h4toh.bias):
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.detach().contiguous())
        out.append(torch.cat(parts, 0).float().requires_grad_(True))
    return out


def _oracle_check(layer, x, gy, world, rank, tol):
    r"""The fused layer against a brute-force fp32 model that owns ALL experts of the group
    (weights all-gathered, its expert gradients summed over ranks): an independent check of
    routing, exchange and GEMMs, in the manner of the reference's distributed tests
    (tests/test_numerical.py:139-202)."""
    act = layer.experts.activation
    layer.zero_grad()
    xx = x.detach().clone().requires_grad_(True)
    y = layer(xx)
    y.backward(gy)
    got = {n: p.grad.detach().float().clone() for n, p in layer.named_parameters()}
    gx = xx.grad.detach().float().clone()
    layer.zero_grad()

    w1, b1, w2, b2 = _gathered_fp32(layer, world)
    x32 = x.detach().float().requires_grad_(True)
    xg = x.detach().clone().requires_grad_(True)
    idx, score = layer.gate(xg)          # the layer's own gate: identical routing decisions
    score32 = score.float()
    ref = torch.zeros_like(x32)
    for j in range(idx.shape[1]):
        for ex in range(w1.shape[0]):
            m = idx[:, j] == ex
            if m.any():
                hid = act(x32[m] @ w1[ex].t() + b1[ex])
                ref[m] = ref[m] + score32[m, j:j + 1] * (hid @ w2[ex].t() + b2[ex])
    ref.backward(gy.float())
    n_exp = layer.num_expert
    for t in (w1, b1, w2, b2):
        g = t.grad if t.grad is not None else torch.zeros_like(t)
        dist.all_reduce(g)
        t.grad = g
    mine = slice(rank * n_exp, (rank + 1) * n_exp)
    assert torch.allclose(y.float(), ref, atol=tol, rtol=tol), float((y.float() - ref).abs().max())
    # the input gradient of the oracle: expert path (x32) plus gate path (xg)
    gx_ref = x32.grad + xg.grad.float()
    assert torch.allclose(gx, gx_ref, atol=2 * tol, rtol=2 * tol), float((gx - gx_ref).abs().max())
    names = ("experts.htoh4.weight", "experts.htoh4.bias", "experts.h4toh.weight", "experts.h4toh.bias")
    for name, t in zip(names, (w1, b1, w2, b2)):
        want = t.grad[mine]
        err = float((got[name] - want).abs().max())
        assert err <= tol * float(want.abs().max()) + 2e-2, (name, err, float(want.abs().max()))
    want = layer.gate.gate.weight.grad.float()
    err = float((got["gate.gate.weight"] - want).abs().max())
    assert err <= 2 * tol * float(want.abs().max()) + 2e-2, ("gate", err)
    assert native.get().read_status(_dev().index) == 0


def case_oracle():
    rank, world = dist.get_rank(), dist.get_world_size()
    cases = ((torch.bfloat16, 2, 2, 512, 256, 512, None, 6e-2),
             (torch.float16, 3, 1, 333, 128, 320, nn.ReLU(), 2e-2),
             (torch.bfloat16, 2, 2, 1200, 256, 1024, nn.GELU(approximate="tanh"), 6e-2),
             # more (peer, expert) pairs than a warp has lanes: the senders decode from memory
             (torch.bfloat16, 40, 2, 900, 128, 256, nn.ReLU(), 6e-2))
    symm.reserve_tokens(dist.group.WORLD, max(c[3] for c in cases), _dev())
    for dtype, num_expert, top_k, n_tok, d, h, act, tol in cases:
        layer = _make_layer(world, rank, num_expert=num_expert, d=d, h=h, top_k=top_k, dtype=dtype,
                            activation=act)
        torch.manual_seed(2000 + rank)
        x = torch.randn(n_tok, d, device=_dev(), dtype=dtype)
        gy = torch.randn(n_tok, d, device=_dev(), dtype=dtype)
        assert symm.fused_available(layer, x), "fused path unavailable"
        _oracle_check(layer, x, gy, world, rank, tol)
    # the in-kernel time stamps of the fused dispatch + GEMM launch
    from fastmoe_b200.utils import profiling
    os.environ["FMOE_EP_TRACE"] = "1"
    with torch.no_grad():
        layer(x)
    del os.environ["FMOE_EP_TRACE"]
    traced = profiling.ep_trace_summary()
    assert len(traced) == 1, traced
    t = traced[0]
    assert t["ctas"] >= 1 and 0 < t["kernel_us"] < 1e6, t
    assert 0 <= t["launch_skew_us"] <= t["kernel_us"], t
    assert t["sender_us"] <= t["kernel_us"] and t["first_rows_us"]["max"] <= t["kernel_us"], t
    assert 0 < t["first_unit_us"]["ids_loaded"] <= t["first_unit_us"]["counted"] <= t["kernel_us"], t
    # the signalling state is back at rest: counters zero, no flag ahead of the epoch, leases back
    del layer
    import gc
    gc.collect()
    dist.barrier()
    report = symm.get_workspace(dist.group.WORLD, _dev()).audit()
    assert report["ok"], report


def case_uneven_tokens():
    r"""Ranks bring different numbers of tokens (and fewer than the agreed budget on later
    calls); the peer-to-peer path must agree with the collective-library path."""
    rank, world = dist.get_rank(), dist.get_world_size()
    layer = _make_layer(world, rank, num_expert=2, top_k=2)
    for call, base in enumerate((700, 500, 640)):
        n_tok = base + 97 * rank - 13 * call * rank
        torch.manual_seed(3000 + 10 * call + rank)
        x = torch.randn(n_tok, 256, device=_dev(), dtype=torch.bfloat16)
        gy = torch.randn(n_tok, 256, device=_dev(), dtype=torch.bfloat16)
        y1, gx1, g1 = _run(layer, x, gy)
        os.environ["FMOE_FUSED"] = "0"
        y2, gx2, g2 = _run(layer, x, gy)
        os.environ["FMOE_FUSED"] = "1"
        assert torch.allclose(y1, y2, atol=2e-2, rtol=2e-2), float((y1 - y2).abs().max())
        assert torch.allclose(gx1, gx2, atol=2e-2, rtol=2e-2)
        for name in g1:
            err = float((g1[name] - g2[name]).abs().max())
            assert err <= 0.04 * float(g2[name].abs().max()) + 1e-3, (name, err)
    # a batch beyond the agreed budget is refused on the host, before any kernel runs
    ws = symm.get_workspace(dist.group.WORLD, _dev())
    too_many = ws.token_budget(1) + 1
    x = torch.randn(too_many, 256, device=_dev(), dtype=torch.bfloat16)
    try:
        layer(x)
        raise AssertionError("a batch beyond the token budget was accepted")
    except RuntimeError as exc:
        assert "reserve_tokens" in str(exc)
    # ... and served after a collective reservation
    symm.reserve_tokens(dist.group.WORLD, too_many + 100 * rank, _dev())
    y = layer(x)
    assert torch.isfinite(y.float()).all()
    assert native.get().read_status(_dev().index) == 0


class _Stack(nn.Module):
    def __init__(self, world, rank, n_layers, d, h):
        super().__init__()
        self.layers = nn.ModuleList([_make_layer(world, rank, d=d, h=h) for _ in range(n_layers)])
        self.norms = nn.ModuleList([nn.LayerNorm(d) for _ in range(n_layers)])

    def forward(self, x):
        for layer, norm in zip(self.layers, self.norms):
            x = x + layer(norm(x))
        return x


def case_multi_layer():
    r"""Three MoE layers back to back (shared return / gradient buffers and flag words, leased
    receive buffers), eager and replayed from a CUDA graph, against the collective-library path."""
    from fastmoe_b200.utils.graph import GraphedStep
    rank, world = dist.get_rank(), dist.get_world_size()
    d, h, n_tok = 256, 512, 768
    model = _Stack(world, rank, 3, d, h).to(_dev()).to(torch.bfloat16)
    torch.manual_seed(4000 + rank)
    xs = [torch.randn(n_tok, d, device=_dev(), dtype=torch.bfloat16) for _ in range(3)]

    def grads_of(x):
        model.zero_grad()
        xx = x.detach().clone().requires_grad_(True)
        y = model(xx)
        y.float().pow(2).mean().backward()
        return ([y.detach().float().clone(), xx.grad.float().clone()]
                + [p.grad.float().clone() for p in model.parameters()])

    # Everything before the capture runs on a side stream as well: autograd binds a parameter's
    # gradient-accumulation node to the stream of its first use, and a node bound to the
    # default stream cannot take part in a capture later.
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fused = [grads_of(x) for x in xs]
        os.environ["FMOE_FUSED"] = "0"
        plain = [grads_of(x) for x in xs]
        os.environ["FMOE_FUSED"] = "1"
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    # Through three layers a rounding difference between the two paths can flip a token's top-k
    # choice in a later layer, so single rows may differ a lot: the paths have to agree on all
    # but a few per cent of the elements ...
    names = ["y", "grad_x"] + [n for n, _ in model.named_parameters()]
    for a, b in zip(fused, plain):
        for name, t, u in zip(names, a, b):
            tol = 0.05 * float(u.abs().max()) + 2e-3
            bad = float(((t - u).abs() > tol).float().mean())
            assert bad <= 0.03, (name, bad)
    # ... and the peer-to-peer path has to reproduce itself bit for bit: a buffer overwritten
    # early or read late by one of the three layers would show up here
    with torch.cuda.stream(side):
        again = [grads_of(x) for x in xs]
    torch.cuda.synchronize()
    for a, b in zip(fused, again):
        for name, t, u in zip(names, a, b):
            if ".gate." in name:   # the gate's weight gradient is summed with fp32 atomics
                assert torch.allclose(t, u, rtol=1e-4, atol=1e-5), (name, float((t - u).abs().max()))
            else:
                assert torch.equal(t, u), (name, float((t - u).abs().max()))

    # the same three-layer step under graph replay: outputs must match the eager fused run
    static_grads = {}

    def step(x):
        model.zero_grad(set_to_none=True)
        xx = x.detach().requires_grad_(True)
        y = model(xx)
        y.float().pow(2).mean().backward()
        static_grads["x"] = xx.grad
        return y

    g = GraphedStep(step, xs[0], warmup=2)
    for i in (1, 2, 0, 1):
        y = g(xs[i]).float()
        torch.cuda.synchronize()
        err = float((y - fused[i][0]).abs().max())
        assert err <= 1e-2 * float(fused[i][0].abs().max()) + 1e-3, (i, err)
        gx = static_grads["x"].float()
        err = float((gx - fused[i][1]).abs().max())
        assert err <= 2e-2 * float(fused[i][1].abs().max()) + 1e-3, (i, err)
    assert native.get().read_status(_dev().index) == 0


def case_exchange_tables():
    r"""The tables the count-exchange kernel leaves on every rank (destination rows, expert
    offsets, the senders' item prefix, the walk order of the row blocks) against the host
    restatement of the same arithmetic on the gathered count matrix; uneven and empty counts, a
    receive buffer that fits and one that clamps."""
    from fastmoe_b200.ops import torch_impl
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = _dev()
    n_expert = 3
    tot = n_expert * world
    symm.reserve_tokens(dist.group.WORLD, 4096, dev)
    ws = symm.get_workspace(dist.group.WORLD, dev)
    for call, capacity in enumerate((4096, 4096, 640)):
        gen = torch.Generator().manual_seed(7000 + 31 * call + rank)
        lec = torch.randint(0, 400, (tot,), generator=gen)
        lec[torch.randint(0, tot, (2,), generator=gen)] = 0
        if call == 1:
            lec = (lec // 100) * 128            # block-aligned boundaries
        lec_dev = lec.to(dev).int()
        tb = symm._Tables(ws, lec_dev, n_expert, capacity)    # pylint: disable=protected-access
        gathered = [torch.empty_like(lec_dev) for _ in range(world)]
        dist.all_gather(gathered, lec_dev)
        mat = torch.stack(gathered).cpu().long()
        dst_base, offs, total, overflow = torch_impl.exchange_offsets(mat, rank, n_expert, capacity)
        assert torch.equal(tb.dst_base.cpu().long(), dst_base), (tb.dst_base, dst_base)
        assert torch.equal(tb.expert_offs.cpu().long(), offs), (tb.expert_offs, offs)
        assert int(tb.total) == total
        prefix = torch_impl.send_item_prefix(mat, rank, n_expert, capacity)
        assert tb.item_prefix.cpu().tolist() == prefix, (tb.item_prefix, prefix)
        order = torch_impl.exchange_block_order(mat, rank, n_expert, capacity)
        got = tb.blk_order.cpu().tolist()[:len(order)]
        assert [(v >> 20, v & 0xFFFFF) for v in got] == order, (got, order)
        status = native.get().read_status(dev.index)
        assert (status != 0) == overflow, (status, overflow)
        if status != 0:
            native.get().clear_status(dev.index)
        dist.barrier()


def case_recv_overflow():
    r"""A bounded receive buffer (FMOE_RECV_CAPACITY_FACTOR) and a gate that sends everything to
    rank 0: rows beyond the capacity are dropped and count as zero, everything that fitted is
    computed as usual (an overflow is a report, not a failure), every rank finds
    STATUS_RECV_OVERFLOW in its status word, and the next, balanced step works after the status
    is cleared."""
    from fastmoe_b200.utils import check_device_status
    nat = native.get()
    rank, world = dist.get_rank(), dist.get_world_size()
    os.environ["FMOE_RECV_CAPACITY_FACTOR"] = "1.0"
    layer = _make_layer(world, rank, num_expert=2, top_k=2)
    torch.manual_seed(5000 + rank)
    x = torch.randn(512, 256, device=_dev(), dtype=torch.bfloat16)
    with torch.no_grad():
        layer.gate.gate.weight.zero_()
        layer.gate.gate.bias.zero_()
        layer.gate.gate.bias[:2] = 10.0      # both experts of rank 0 win every token
    y = layer(x)
    torch.cuda.synchronize()
    assert torch.isfinite(y.float()).all()
    if world == 2:
        # every token picks experts 0 and 1 with score 1/2 each; expert 0's segment on rank 0
        # is exactly the buffer (2 x 512 rows), expert 1's lies beyond it: y = expert0(x) / 2
        ex = layer.experts
        w1, b1 = ex.htoh4.weight.detach()[0].clone(), ex.htoh4.bias.detach()[0].clone()
        w2, b2 = ex.h4toh.weight.detach()[0].clone(), ex.h4toh.bias.detach()[0].clone()
        for t in (w1, b1, w2, b2):
            dist.broadcast(t, 0)
        hid = torch.nn.functional.gelu(x.float() @ w1.float().t() + b1.float())
        want = 0.5 * (hid.to(x.dtype).float() @ w2.float().t() + b2.float())
        err = float((y.detach().float() - want).abs().max())
        assert err <= 3e-2 * float(want.abs().max()) + 1e-2, err
    try:
        check_device_status(_dev())
        raise AssertionError("overflow was not reported")
    except RuntimeError as exc:
        assert str(nat.STATUS_RECV_OVERFLOW) in str(exc), str(exc)
    dist.barrier()
    # a near-uniform gate and a buffer with 60 % head-room: nothing is dropped any more
    os.environ["FMOE_RECV_CAPACITY_FACTOR"] = "1.6"
    with torch.no_grad():
        layer.gate.gate.bias.zero_()
        layer.gate.gate.weight.normal_(0, 0.02)
    gy = torch.randn_like(x)
    y1, gx1, _ = _run(layer, x, gy)
    os.environ["FMOE_FUSED"] = "0"
    y2, gx2, _ = _run(layer, x, gy)
    os.environ["FMOE_FUSED"] = "1"
    assert check_device_status(_dev()) == 0
    del os.environ["FMOE_RECV_CAPACITY_FACTOR"]
    # balanced routing fits into the bounded buffer with probability ~1 only when nothing is
    # dropped; compare where the bounded run kept everything
    if float((y1 - y2).abs().max()) > 2e-2:
        raise AssertionError("balanced step after the overflow differs: %g" % float((y1 - y2).abs().max()))


def case_allreduce():
    rank, world = dist.get_rank(), dist.get_world_size()
    for dtype in (torch.bfloat16, torch.float32):
        torch.manual_seed(rank)
        grads = [torch.randn(1000, 37, device=_dev()).to(dtype), torch.randn(5, device=_dev()).to(dtype)]
        ref = [g.float().clone() for g in grads]
        for r in ref:
            dist.all_reduce(r)
        ok = symm.allreduce_grads(grads, dist.group.WORLD, 1.0 / world)
        assert ok
        for g, r in zip(grads, ref):
            assert torch.allclose(g.float(), r / world, atol=2e-2, rtol=2e-2)
        # bit-identical on all ranks
        mine = grads[0].float()
        other = mine.clone()
        dist.broadcast(other, 0)
        assert torch.equal(mine, other)
    # a bucket large enough for the two-shot kernel, with a ragged element count
    for dtype in (torch.bfloat16, torch.float32):
        torch.manual_seed(100 + rank)
        grads = [torch.randn(2048, 1537, device=_dev()).to(dtype), torch.randn(3, device=_dev()).to(dtype)]
        nbytes = sum(g.numel() for g in grads) * grads[0].element_size()
        assert symm._two_shot(nbytes, world)  # pylint: disable=protected-access
        ref = [g.float().clone() for g in grads]
        for r in ref:
            dist.all_reduce(r)
        assert symm.allreduce_grads(grads, dist.group.WORLD, 1.0 / world)
        for g, r in zip(grads, ref):
            assert torch.allclose(g.float(), r / world, atol=2e-2, rtol=2e-2)
        mine = grads[0].float()
        other = mine.clone()
        dist.broadcast(other, 0)
        assert torch.equal(mine, other)
        assert native.get().read_status(_dev().index) == 0


def case_allreduce_nvls():
    r"""The NVSwitch (multimem) all-reduce against the collective library; skipped with a note
    when the symmetric allocation has no multicast mapping on this machine."""
    rank, world = dist.get_rank(), dist.get_world_size()
    os.environ["FMOE_USE_NVLS"] = "1"
    ws = symm.get_workspace(dist.group.WORLD, _dev())
    ws.buffer("allreduce", 1 << 20)
    if ws.multicast_ptr("allreduce") == 0:
        print("no multicast mapping on this machine: NVLS path not exercised")
        return
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        for numel in (1000 * 37 + 5, 2048 * 1537 + 3):
            torch.manual_seed(200 + rank)
            flat = torch.randn(numel, device=_dev()).to(dtype)
            ref = flat.float().clone()
            dist.all_reduce(ref)
            got = symm.allreduce_flat(flat, dist.group.WORLD, 1.0 / world)
            assert got is not None
            assert torch.allclose(got.float(), ref / world, atol=2e-2, rtol=2e-2), \
                (dtype, numel, float((got.float() - ref / world).abs().max()))
            other = got.float().clone()
            dist.broadcast(other, 0)
            assert torch.equal(got.float(), other)          # bit-identical on all ranks
    del os.environ["FMOE_USE_NVLS"]
    assert native.get().read_status(_dev().index) == 0


def case_grouped_ddp():
    rank, world = dist.get_rank(), dist.get_world_size()
    layer = _make_layer(world, rank)
    model = DistributedGroupedDataParallel(layer)
    torch.manual_seed(50 + rank)
    x = torch.randn(256, 256, device=_dev(), dtype=torch.bfloat16)
    model(x).float().pow(2).mean().backward()
    local = layer.gate.gate.weight.grad.float().clone()
    expert_before = layer.experts.htoh4.weight.grad.clone()
    model.allreduce_params()
    ref = local.clone()
    dist.all_reduce(ref)
    assert torch.allclose(layer.gate.gate.weight.grad.float(), ref / world, atol=1e-2, rtol=2e-2)
    assert torch.equal(layer.experts.htoh4.weight.grad, expert_before)
    # the same reduction issued on the side stream, with unrelated work queued in between
    layer.gate.gate.weight.grad.copy_(local.to(layer.gate.gate.weight.grad.dtype))
    pending = model.allreduce_params(async_op=True)
    busy = expert_before.float().square().sum()
    pending.wait()
    torch.cuda.synchronize()
    assert torch.allclose(layer.gate.gate.weight.grad.float(), ref / world, atol=1e-2, rtol=2e-2)
    assert torch.isfinite(busy)


def case_slice_group():
    r"""Peer-to-peer all-gather (rows of every rank in rank order), then a layer with
    ``slice_group``: ranks share the input, each routes its slice, outputs are all-gathered."""
    from fastmoe_b200.functions import AllGather, Slice
    rank, world = dist.get_rank(), dist.get_world_size()
    for rows, cols, dtype in ((5, 24, torch.bfloat16), (300, 256, torch.float32)):
        torch.manual_seed(3 + rank)
        mine = torch.randn(rows, cols, device=_dev()).to(dtype)
        got = symm.allgather_rows(mine, dist.group.WORLD)
        assert got is not None
        ref = torch.empty(world * rows, cols, device=_dev(), dtype=dtype)
        dist.all_gather_into_tensor(ref, mine)
        assert torch.equal(got, ref)
    # differentiable wrappers: AllGather backward keeps the own slice, Slice backward gathers
    torch.manual_seed(8)
    full = torch.randn(8 * world, 16, device=_dev(), requires_grad=True)
    part = Slice.apply(full, rank, world, dist.group.WORLD)
    back = AllGather.apply(part * (rank + 1.0), rank, world, dist.group.WORLD)
    scale = torch.arange(1, world + 1, device=_dev(), dtype=torch.float32).repeat_interleave(8)[:, None]
    assert torch.allclose(back, full.detach() * scale)
    back.sum().backward()
    assert torch.allclose(full.grad, torch.ones_like(full) * scale)
    torch.manual_seed(9)
    moe = FMoETransformerMLP(num_expert=2, d_model=256, d_hidden=512, world_size=1, top_k=2,
                             slice_group=dist.group.WORLD).to(_dev()).to(torch.bfloat16)
    ref_layer = FMoETransformerMLP(num_expert=2, d_model=256, d_hidden=512, world_size=1,
                                   top_k=2).to(_dev()).to(torch.bfloat16)
    ref_layer.load_state_dict(moe.state_dict())
    x = torch.randn(64 * world, 256, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    y = moe(x)
    ref = ref_layer(x.detach())
    assert torch.allclose(y.float(), ref.float(), atol=3e-2, rtol=3e-2)
    y.float().sum().backward()
    assert x.grad.shape == x.shape
    assert native.get().read_status(_dev().index) == 0


def case_capacity():
    r"""Global capacity limit: the single-exchange grant kernel against the two all-to-alls of
    the collective-library path, including per-rank capacities that differ."""
    from fastmoe_b200.functions import ensure_comm
    from fastmoe_b200.gates.utils import limit_by_capacity
    rank, world = dist.get_rank(), dist.get_world_size()
    ensure_comm(torch.zeros(1, device=_dev()), None)
    n_expert = 3
    for trial in range(3):
        torch.manual_seed(40 + 7 * trial + rank)
        idx = torch.randint(0, n_expert * world, (257 + 13 * rank, 2), device=_dev())
        capacity = 40 + 5 * trial + (3 * rank if trial == 2 else 0)
        os.environ["FMOE_FUSED"] = "1"
        a_lec, a_gec, a_idx = limit_by_capacity(idx.clone(), n_expert, world, capacity)
        os.environ["FMOE_FUSED"] = "0"
        b_lec, b_gec, b_idx = limit_by_capacity(idx.clone(), n_expert, world, capacity)
        os.environ["FMOE_FUSED"] = "1"
        assert torch.equal(a_lec.long(), b_lec.long()), (a_lec, b_lec)
        assert torch.equal(a_gec.long(), b_gec.long())
        assert torch.equal(a_idx, b_idx)
        assert int(a_gec.view(world, n_expert).sum(0).max()) <= capacity
    assert native.get().read_status(_dev().index) == 0


def case_wait_timeout():
    r"""A device wait on a flag that nothing sets returns after its limit with a status code;
    the context stays usable."""
    nat = native.get()
    ws = symm.get_workspace(dist.group.WORLD, _dev())
    assert ws is not None
    ws.set_timeout_ms(300)
    ws.ctx.wait_only(nat.P2P_CHAN_RETURN)
    torch.cuda.synchronize()
    assert nat.read_status(_dev().index) == nat.STATUS_PEER_TIMEOUT
    nat.clear_status(_dev().index)
    ws.set_timeout_ms(4000)
    dist.barrier()
    # the exchange still works afterwards
    case_allreduce()
    assert nat.read_status(_dev().index) == 0


def case_smart_schedule():
    r"""FasterMoE smart schedule with shadow experts on GPUs (NCCL exchange on a side stream,
    bf16 backward) against the plain general path."""
    from fastmoe_b200.fastermoe import schedule
    from fastmoe_b200.functions import ensure_comm
    from fastmoe_b200.layers import _fmoe_general_global_forward as naive_forward
    rank, world = dist.get_rank(), dist.get_world_size()
    ensure_comm(torch.zeros(1, device=_dev()), None)
    for dtype in (torch.float32, torch.bfloat16):
        for group_size, shadow in ((1, False), (2, True)):
            os.environ["FMOE_FASTER_GROUP_SIZE"] = str(group_size)
            layer = _make_layer(world, rank, num_expert=2, d=128, h=256, dtype=dtype)
            torch.manual_seed(300 + rank)
            x = torch.randn(200 + 8 * rank, 128, device=_dev(), dtype=dtype)
            idx = torch.randint(0, 2 * world, (x.shape[0], 2), device=_dev())
            torch.manual_seed(77)
            stored = torch.rand(2 * world) < 0.5 if shadow else torch.zeros(2 * world, dtype=torch.bool)

            xa = x.clone().requires_grad_(True)
            ya = naive_forward(xa, idx, layer.expert_fn, 2, world)
            ya.float().pow(2).sum().backward()
            ga = [p.grad.float().clone() for p in layer.experts.parameters()]
            layer.zero_grad()
            xb = x.clone().requires_grad_(True)
            yb = schedule._fmoe_general_global_forward(
                xb, idx, layer.expert_fn_single, 2, world, experts=layer.experts, stored_models=stored)
            yb.float().pow(2).sum().backward()
            gb = [p.grad.float().clone() for p in layer.experts.parameters()]
            tol = 1e-3 if dtype == torch.float32 else 4e-2
            assert torch.allclose(ya.float(), yb.float(), atol=tol, rtol=tol), (dtype, shadow)
            assert torch.allclose(xa.grad.float(), xb.grad.float(), atol=tol * 4, rtol=tol * 2)
            for a, b in zip(ga, gb):
                assert float((a - b).abs().max()) <= 0.05 * float(a.abs().max()) + 1e-3


def case_shadow_fused():
    r"""Shadow experts on the fused path: masked out of the exchange, parameters pushed by their
    owners, computed locally, gradients reduced to the owners — against the plain fused path."""
    from fastmoe_b200.fastermoe import fused_shadow
    from fastmoe_b200.ops import fused
    rank, world = dist.get_rank(), dist.get_world_size()
    n_exp = 2
    layer = _make_layer(world, rank, num_expert=n_exp, d=256, h=512, top_k=2)
    torch.manual_seed(6000 + rank)
    x = torch.randn(600 + 16 * rank, 256, device=_dev(), dtype=torch.bfloat16)
    gy = torch.randn_like(x)
    stored = torch.zeros(world * n_exp, dtype=torch.bool)
    stored[1] = True                      # expert 1 of rank 0
    stored[(world - 1) * n_exp] = True    # expert 0 of the last rank
    symm.reserve_tokens(dist.group.WORLD, 600 + 16 * world, _dev())

    def run(fn):
        layer.zero_grad()
        xx = x.detach().clone().requires_grad_(True)
        idx, score = layer.gate(xx)
        y = fn(layer, xx, idx, score)
        y.backward(gy)
        return (y.detach().float(), xx.grad.float().clone(),
                {n: p.grad.float().clone() for n, p in layer.named_parameters()})

    y0, gx0, g0 = run(fused.moe_mlp_forward)
    y1, gx1, g1 = run(lambda l, a, i, sc: fused_shadow.moe_mlp_forward(l, a, i, sc, stored=stored))
    assert torch.allclose(y0, y1, atol=3e-2, rtol=3e-2), float((y0 - y1).abs().max())
    assert torch.allclose(gx0, gx1, atol=3e-2, rtol=3e-2), float((gx0 - gx1).abs().max())
    for name in g0:
        err = float((g0[name] - g1[name]).abs().max())
        assert err <= 0.04 * float(g0[name].abs().max()) + 2e-3, (name, err)
    # the policy-driven entry (whatever it decides) must agree as well
    os.environ["FMOE_FASTER_SCHEDULE_ENABLE"] = "1"
    os.environ["FMOE_FASTER_SHADOW_ENABLE"] = "1"
    y2, _gx2, _g2 = run(lambda l, a, i, sc: fused_shadow.moe_mlp_forward(l, a, i, sc))
    del os.environ["FMOE_FASTER_SCHEDULE_ENABLE"], os.environ["FMOE_FASTER_SHADOW_ENABLE"]
    assert torch.allclose(y0, y2, atol=3e-2, rtol=3e-2)
    assert native.get().read_status(_dev().index) == 0


def case_swipe_device():
    r"""SWIPE rounds computed by the device kernels (exchange + plan + reassignment, no host read)
    against the all-gather + host plan; then a SwipeGate forward in training mode."""
    from fastmoe_b200 import gates
    from fastmoe_b200.functions import ensure_comm
    from fastmoe_b200.ops import api
    rank, world = dist.get_rank(), dist.get_world_size()
    ensure_comm(torch.zeros(1, device=_dev()), None)
    n_expert = 3
    for trial in range(4):
        torch.manual_seed(700 + 11 * trial + rank)
        n = 500 + 37 * rank
        # skewed preferences: most tokens want worker 0
        idx = torch.randint(0, n_expert * world, (n,), device=_dev())
        idx = torch.where(torch.rand(n, device=_dev()) < 0.6, idx % n_expert, idx)
        cap = torch.tensor([n * 2 - 100 * trial], dtype=torch.long, device=_dev())
        os.environ["FMOE_FUSED"] = "1"
        a_idx, a_left = api.swipe_once(idx, cap, n_expert, world, trial % n_expert)
        assert a_idx.is_cuda and a_left.is_cuda
        os.environ["FMOE_FUSED"] = "0"
        b_idx, b_left = api.swipe_once(idx, cap, n_expert, world, trial % n_expert)
        os.environ["FMOE_FUSED"] = "1"
        assert torch.equal(a_idx.cpu(), b_idx.cpu()), (trial, int((a_idx.cpu() != b_idx.cpu()).sum()))
        assert int(a_left.cpu()) == int(b_left), (int(a_left.cpu()), int(b_left))
    gate = gates.SwipeGate(64, n_expert, world, top_k=2).to(_dev())
    gate.train()
    x = torch.randn(256, 64, device=_dev())
    ids, score = gate(x)
    assert ids.shape == (256, 2) and torch.isfinite(score).all()
    loads = torch.bincount(torch.div(ids.reshape(-1), n_expert, rounding_mode="floor").clamp_min(0),
                           minlength=world).float()
    dist.all_reduce(loads)
    assert float(loads.max()) <= 256 * 2 + 1e-3      # no worker takes more than B * top_k tokens
    assert native.get().read_status(_dev().index) == 0


def case_pipeline_gpu():
    r"""Pipeline parallelism on GPUs: the 1F1B runner with one stage per GPU (NCCL send / recv
    between stages, the fused single-GPU MoE kernels inside a stage, bf16) against the same
    model run in one process."""
    from fastmoe_b200.parallel.pipeline import PipelineRunner, build_stage_groups
    rank, world = dist.get_rank(), dist.get_world_size()
    n_stages, n_micro, tokens, d, h, n_exp, blocks = world, 3, 128, 256, 512, 2, 2
    stage, group, prev_rank, next_rank = build_stage_groups(n_stages)
    dev = _dev()

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = nn.Linear(d, d)
            self.moe = FMoETransformerMLP(num_expert=n_exp, d_model=d, d_hidden=h, top_k=2, world_size=1)

        def forward(self, x):
            return x + self.moe(torch.tanh(self.lin(x)))

    torch.manual_seed(17)
    full = nn.Sequential(*[Block() for _ in range(n_stages * blocks)]).to(dev).to(torch.bfloat16)
    mine = nn.Sequential(*[Block() for _ in range(blocks)]).to(dev).to(torch.bfloat16)
    refs = list(full)[stage * blocks:(stage + 1) * blocks]
    for b, ref in zip(mine, refs):
        b.load_state_dict(ref.state_dict())
    gen = torch.Generator().manual_seed(300)
    xs = [torch.randn(tokens, d, generator=gen).to(dev).to(torch.bfloat16) for _ in range(n_micro)]
    ts = [torch.randn(tokens, d, generator=gen).to(dev).to(torch.bfloat16) for _ in range(n_micro)]

    def mse(out, target):
        return (out.float() - target.float()).pow(2).mean()

    runner = PipelineRunner(mine, stage, n_stages, prev_rank, next_rank, (tokens, d), torch.bfloat16,
                            loss_fn=mse, device=dev)
    loss = runner.run(micro_batches=xs if stage == 0 else None,
                      targets=ts if stage == n_stages - 1 else None, n_micro=n_micro)
    total = 0.0
    for x, t in zip(xs, ts):
        total = total + mse(full(x), t) / n_micro
    total.backward()
    if stage == n_stages - 1:
        assert abs(float(loss) - float(total)) <= 2e-2 * abs(float(total)) + 1e-3, (float(loss), float(total))
    for b, ref in zip(mine, refs):
        for (name, p), (_n, q) in zip(b.named_parameters(), ref.named_parameters()):
            err = float((p.grad.float() - q.grad.float()).abs().max())
            assert err <= 0.06 * float(q.grad.float().abs().max()) + 2e-3, (name, err)
    assert native.get().read_status(dev.index) == 0


def case_graph_step():
    r"""A whole expert-parallel training step replays from a CUDA graph."""
    from fastmoe_b200.utils.graph import GraphedStep
    rank, world = dist.get_rank(), dist.get_world_size()
    layer = _make_layer(world, rank)
    model = DistributedGroupedDataParallel(layer)
    opt = torch.optim.Adam(layer.parameters(), lr=1e-3, fused=True, capturable=True)

    def step(x):
        opt.zero_grad(set_to_none=True)
        loss = model(x).float().pow(2).mean()
        loss.backward()
        model.allreduce_params()
        opt.step()
        return loss

    torch.manual_seed(60 + rank)
    x = torch.randn(512, 256, device=_dev(), dtype=torch.bfloat16)
    g = GraphedStep(step, x, warmup=3)
    losses = [float(g(x)) for _ in range(5)]
    assert all(l == l for l in losses)
    assert losses[-1] < losses[0], losses
    assert native.get().read_status(_dev().index) == 0


if __name__ == "__main__":
    case = sys.argv[1]
    torch.cuda.set_device(_dev())
    dist.init_process_group("nccl", device_id=_dev())
    globals()["case_" + case]()
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
