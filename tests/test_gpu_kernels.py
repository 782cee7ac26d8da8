r"""GPU tier: every sm_100a kernel against a plain PyTorch fp32 restatement of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _native():
    from fastmoe_b200.ops import native
    return native.get()


def _offs(counts):
    o = torch.zeros(len(counts) + 1, dtype=torch.int32)
    o[1:] = torch.cumsum(torch.tensor(counts), 0)
    return o.to(DEV)


def _segments(counts):
    base = 0
    for e, n in enumerate(counts):
        yield e, base, base + n
        base += n


def _tiled(pre, offs, groups):
    r"""Tile-blocked copy of a row-major pre-activation: the inverse of ``gg.untile_pre``."""
    from fastmoe_b200.ops import grouped_gemm as gg
    rows, n = pre.shape
    buf = gg.pre_buffer(rows, n, groups, pre.dtype, pre.device).zero_()
    blocks = buf.view(-1, 2, 4, 4, 4, 32, 8)     # tile, half, part, chunk, piece, lane, v
    o = [int(v) for v in offs.tolist()]
    n_tiles = (n + gg.TILE_N - 1) // gg.TILE_N
    tile = 0
    for e in range(groups):
        for m in range((o[e + 1] - o[e] + gg.TILE_M - 1) // gg.TILE_M):
            for nt in range(n_tiles):
                full = torch.zeros(gg.TILE_M, gg.TILE_N, dtype=pre.dtype, device=pre.device)
                r0, c0 = o[e] + m * gg.TILE_M, nt * gg.TILE_N
                nr, nc = min(gg.TILE_M, o[e + 1] - r0), min(gg.TILE_N, n - c0)
                full[:nr, :nc] = pre[r0:r0 + nr, c0:c0 + nc]
                blocks[tile] = full.view(4, 32, 2, 4, 4, 8).permute(2, 0, 3, 4, 1, 5)
                tile += 1
    return buf


def _tol(dtype, k):
    # bf16 has 8 bits of mantissa: inputs are exact in fp32, the only error is the output rounding.
    return (2e-2 if dtype == torch.bfloat16 else 4e-3)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("counts,k,n", [
    ([100, 200], 64, 32),
    ([128, 0, 257, 5], 128, 256),
    ([300, 1, 511], 256, 320),
    ([1000, 24], 1024, 512),
    ([513, 130], 4096, 96),
])
def test_grouped_gemm_forward(dtype, counts, k, n):
    from fastmoe_b200.ops import grouped_gemm as gg
    torch.manual_seed(0)
    rows = sum(counts)
    pad = 7  # rows past the last segment must stay untouched
    x = torch.randn(rows + pad, k, device=DEV, dtype=dtype)
    w = (torch.randn(len(counts), n, k, device=DEV) / k ** 0.5).to(dtype)
    b = torch.randn(len(counts), n, device=DEV).to(dtype)
    offs = _offs(counts)
    out, pre = gg.forward(x, w, offs, b, act="gelu", want_pre=True)
    if pre.dim() == 1:
        pre = gg.untile_pre(pre, offs, n, x.shape[0])
    for e, lo, hi in _segments(counts):
        ref_pre = x[lo:hi].float() @ w[e].float().t() + b[e].float()
        ref = torch.nn.functional.gelu(ref_pre)
        assert torch.allclose(pre[lo:hi].float(), ref_pre, atol=_tol(dtype, k), rtol=2e-2)
        assert torch.allclose(out[lo:hi].float(), ref, atol=_tol(dtype, k), rtol=2e-2)
    assert _native().read_status(0) == 0


@pytest.mark.parametrize("act", [None, "relu", "gelu_tanh"])
@pytest.mark.parametrize("counts,k,n", [([70, 300, 129], 192, 448), ([2048, 2048], 4096, 1024)])
def test_grouped_gemm_epilogues(act, counts, k, n):
    r"""The other fused epilogues, forward and input gradient, including a span of columns that
    is not a multiple of the 256-column tile and a K of 4096."""
    from fastmoe_b200.ops import grouped_gemm as gg
    torch.manual_seed(5)
    dtype = torch.bfloat16
    rows = sum(counts)
    x = torch.randn(rows, k, device=DEV, dtype=dtype)
    w = (torch.randn(len(counts), n, k, device=DEV) / k ** 0.5).to(dtype)
    b = torch.randn(len(counts), n, device=DEV).to(dtype)
    offs = _offs(counts)
    out, pre = gg.forward(x, w, offs, b, act=act, want_pre=True)
    if pre.dim() == 1:
        pre = gg.untile_pre(pre, offs, n, rows)
    fn = {None: lambda t: t, "relu": torch.relu,
          "gelu_tanh": lambda t: torch.nn.functional.gelu(t, approximate="tanh")}[act]
    dy = torch.randn(rows, n, device=DEV, dtype=dtype)
    wt = (torch.randn(len(counts), n, k, device=DEV) / n ** 0.5).to(dtype)   # [E, k(out)=n, n(in)=k]
    pre_in = torch.randn(rows, k, device=DEV, dtype=dtype)
    dx = gg.dgrad(dy, wt, offs, pre=_tiled(pre_in, offs, len(counts)) if act else None, act=act)
    p32 = pre_in.float().requires_grad_(True)
    fn(p32).sum().backward()
    for e, lo, hi in _segments(counts):
        ref_pre = x[lo:hi].float() @ w[e].float().t() + b[e].float()
        assert torch.allclose(pre[lo:hi].float(), ref_pre, atol=2e-2, rtol=2e-2)
        assert torch.allclose(out[lo:hi].float(), fn(ref_pre), atol=2e-2, rtol=2e-2)
        ref_dx = dy[lo:hi].float() @ wt[e].float()
        if act:
            ref_dx = ref_dx * p32.grad[lo:hi]
        assert torch.allclose(dx[lo:hi].float(), ref_dx, atol=2e-2, rtol=2e-2)
    assert _native().read_status(0) == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("counts,k,n", [
    ([100, 200], 64, 64),
    ([128, 0, 257, 5], 256, 128),
    ([700, 324], 512, 1024),
])
def test_grouped_gemm_dgrad(dtype, counts, k, n):
    r"""dX = (dY W) * gelu'(pre) with W stored [E, k(out), n(in)]."""
    from fastmoe_b200.ops import grouped_gemm as gg
    torch.manual_seed(1)
    rows = sum(counts)
    dy = torch.randn(rows, k, device=DEV, dtype=dtype)
    w = (torch.randn(len(counts), k, n, device=DEV) / k ** 0.5).to(dtype)
    pre = torch.randn(rows, n, device=DEV, dtype=dtype)
    offs = _offs(counts)
    plain = gg.dgrad(dy, w, offs)
    fused = gg.dgrad(dy, w, offs, pre=_tiled(pre, offs, len(counts)), act="gelu")
    rowmajor = gg.dgrad(dy, w, offs, pre=pre, act="gelu")   # plain matrix: derivative as a PyTorch op
    assert torch.allclose(rowmajor[:rows].float(), fused[:rows].float(), atol=2e-2, rtol=2e-2)
    p32 = pre.float().requires_grad_(True)
    torch.nn.functional.gelu(p32).sum().backward()
    for e, lo, hi in _segments(counts):
        ref = dy[lo:hi].float() @ w[e].float()
        assert torch.allclose(plain[lo:hi].float(), ref, atol=_tol(dtype, k), rtol=2e-2)
        assert torch.allclose(fused[lo:hi].float(), ref * p32.grad[lo:hi], atol=_tol(dtype, k), rtol=2e-2)
    assert _native().read_status(0) == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("counts,m,n", [
    ([64, 128], 128, 256),
    ([100, 0, 37, 300], 64, 32),
    ([1000, 24, 513], 256, 512),
])
def test_grouped_gemm_wgrad(dtype, counts, m, n):
    from fastmoe_b200.ops import grouped_gemm as gg
    torch.manual_seed(2)
    rows = sum(counts)
    pad = 70  # garbage rows after the last segment must not leak into the last expert
    dy = torch.randn(rows + pad, m, device=DEV, dtype=dtype)
    x = torch.randn(rows + pad, n, device=DEV, dtype=dtype)
    dy[rows:] = float("nan")
    x[rows:] = float("nan")
    offs = _offs(counts)
    out = gg.wgrad(dy, x, offs, len(counts))
    for e, lo, hi in _segments(counts):
        ref = dy[lo:hi].float().t() @ x[lo:hi].float()
        scale = max(1.0, (hi - lo) ** 0.5)
        assert torch.allclose(out[e].float(), ref, atol=_tol(dtype, hi - lo) * scale, rtol=2e-2), e
    bg = gg.bias_grad(dy[:rows].contiguous(), offs)
    for e, lo, hi in _segments(counts):
        ref = dy[lo:hi].float().sum(0)
        assert torch.allclose(bg[e].float(), ref, atol=0.3, rtol=2e-2)
    # the same sums produced inside the weight-gradient kernel, with and without accumulation
    out2, bg2 = gg.wgrad(dy, x, offs, len(counts), with_bias_grad=True)
    assert torch.equal(out2, out)
    for e, lo, hi in _segments(counts):
        ref = dy[lo:hi].float().sum(0)
        assert torch.allclose(bg2[e].float(), ref, atol=0.3, rtol=2e-2), e
    if gg._tc_ok(dy, gg.MODE_WGRAD, m, n, 0, len(counts)):
        acc_w = out.clone()
        acc_b = bg2.clone()
        _native().grouped_gemm(gg.MODE_WGRAD, dy, x, offs, acc_w, None, None, None, 0, 0, True, acc_b)
        assert torch.allclose(acc_b.float(), 2 * bg2.float(), atol=0.6, rtol=3e-2)
        for e, lo, hi in _segments(counts):
            scale = max(1.0, (hi - lo) ** 0.5)
            assert torch.allclose(acc_w[e].float(), 2 * out[e].float(), atol=_tol(dtype, 0) * 2 * scale,
                                  rtol=3e-2), e
        acc32 = torch.ones(len(counts), m, n, device=DEV, dtype=torch.float32)
        _native().grouped_gemm(gg.MODE_WGRAD, dy, x, offs, acc32, None, None, None, 0, 0, True, None)
        for e, lo, hi in _segments(counts):
            ref = 1.0 + dy[lo:hi].float().t() @ x[lo:hi].float()
            assert torch.allclose(acc32[e], ref, atol=1e-2 * max(1.0, (hi - lo) ** 0.5), rtol=1e-2), e
    assert _native().read_status(0) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("counts,k,n", [([5, 0, 9, 3], 16, 24), ([300, 65, 0, 130], 200, 150)])
def test_simt_grouped_linear(dtype, counts, k, n):
    r"""The shared-memory tiled kernel for fp32 / fp64, ragged in every dimension."""
    from fastmoe_b200.ops import grouped_gemm as gg
    torch.manual_seed(3)
    torch.backends.cuda.matmul.allow_tf32 = False
    rows = sum(counts)
    x = torch.randn(rows, k, device=DEV, dtype=dtype)
    w = torch.randn(len(counts), n, k, device=DEV, dtype=dtype)
    b = torch.randn(len(counts), n, device=DEV, dtype=dtype)
    go = torch.randn(rows, n, device=DEV, dtype=dtype)
    cnt = torch.tensor(counts)
    out = gg.linear_forward_host_counts(x, cnt, w, b)
    gi, gw, gb = gg.linear_backward_host_counts(go, x, cnt, w, b)
    for e, lo, hi in _segments(counts):
        assert torch.allclose(out[lo:hi], x[lo:hi] @ w[e].t() + b[e], atol=2e-3, rtol=1e-4)
        assert torch.allclose(gi[lo:hi], go[lo:hi] @ w[e], atol=2e-3, rtol=1e-4)
        assert torch.allclose(gw[e], go[lo:hi].t() @ x[lo:hi], atol=2e-3, rtol=1e-4)
        assert torch.allclose(gb[e], go[lo:hi].sum(0), atol=2e-3, rtol=1e-4)


@pytest.mark.parametrize("n_slots,tot", [(7, 3), (64, 4), (8192, 16), (50001, 64), (4096, 1024),
                                         (1000003, 256), (300000, 8)])
def test_route_matches_cpu(n_slots, tot):
    r"""Counts, ranks, offsets and the sorted slot list; above 32 K slots several CTAs share the
    ranking (two launches) and must reproduce the single ordered scan."""
    from fastmoe_b200.ops import torch_impl
    torch.manual_seed(4)
    idx = torch.randint(-1, tot, (n_slots,), device=DEV)
    counts, rank, offs = _native().route_offs(idx, tot)
    c2, r2, o2, pos = _native().route_pos(idx, tot)
    assert torch.equal(c2, counts) and torch.equal(r2, rank) and torch.equal(o2, offs)
    kept = int(offs[-1])
    order = torch.argsort(torch.where(idx >= 0, idx, tot).cpu(), stable=True)[:kept]
    assert torch.equal(pos[:kept].cpu().long(), order)
    ref_counts = torch_impl.expert_count(idx.cpu(), tot)
    ref_rank = torch_impl.slot_rank(idx.cpu(), tot)
    assert torch.equal(counts.cpu(), ref_counts)
    assert torch.equal(rank.cpu().long(), ref_rank)
    assert torch.equal(offs.cpu()[1:].long(), torch.cumsum(ref_counts.long(), 0))


def test_capacity_kernels_match_cpu():
    from fastmoe_b200.ops import api, torch_impl
    torch.manual_seed(5)
    n_expert, n_worker = 4, 3
    ec = torch.randint(0, 20, (n_expert * n_worker,), dtype=torch.int64)
    cap = torch.full((n_expert,), 25, dtype=torch.int32)
    ref = torch_impl.limit_by_capacity(ec.clone(), cap.clone(), n_expert, n_worker)
    cap_d = cap.to(DEV)
    got = api.limit_by_capacity(ec.to(DEV), cap_d, n_expert, n_worker)
    assert torch.equal(got.cpu(), ref)
    idx = torch.randint(-1, n_expert * n_worker, (100, 2))
    capg = torch.randint(0, 12, (n_expert * n_worker,), dtype=torch.int32)
    ref_idx = torch_impl.prune_gate_by_capacity(idx.clone(), capg.clone(), n_expert, n_worker)
    got_idx = api.prune_gate_by_capacity(idx.to(DEV), capg.to(DEV), n_expert, n_worker)
    assert torch.equal(got_idx.cpu(), ref_idx)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_scatter_combine_roundtrip(dtype):
    torch.manual_seed(6)
    nat = _native()
    n_tok, k, d, tot = 300, 2, 256, 8
    x = torch.randn(n_tok, d, device=DEV, dtype=dtype)
    idx = torch.randint(-1, tot, (n_tok * k,), device=DEV)
    score = torch.rand(n_tok * k, device=DEV).to(dtype)
    counts, rank, offs = nat.route_offs(idx, tot)
    rows = torch.full((n_tok * k, d), float("nan"), device=DEV, dtype=dtype)
    row_slot = torch.full((n_tok * k,), -1, device=DEV, dtype=torch.int32)
    nat.scatter_rows(x, idx, rank, offs, None, k, rows, row_slot)
    n_valid = int(offs[-1])
    slots = row_slot[:n_valid].long()
    assert torch.equal(rows[:n_valid], x[slots // k])
    # rows are grouped by expert, ascending slot inside an expert
    assert torch.equal(idx[slots], torch.sort(idx[idx >= 0], stable=True).values)
    out = torch.empty(n_tok, d, device=DEV, dtype=dtype)
    nat.gather_combine(rows, idx, rank, offs, score, k, out)
    w = torch.where(idx >= 0, score.float(), torch.zeros_like(score, dtype=torch.float32))
    ref = (x.float().repeat_interleave(k, 0) * w[:, None]).view(n_tok, k, d).sum(1)
    assert torch.allclose(out.float(), ref, atol=3e-2, rtol=2e-2)
    # backward of the weighted combine
    dout = torch.randn(n_tok, d, device=DEV, dtype=dtype)
    drows = torch.zeros_like(rows)
    dscore = torch.empty(n_tok * k, device=DEV, dtype=dtype)
    nat.combine_bwd(dout, rows, idx, rank, offs, score, k, drows, dscore)
    ref_ds = (dout.float().repeat_interleave(k, 0) * x.float().repeat_interleave(k, 0)).sum(1)
    ref_ds = torch.where(idx >= 0, ref_ds, torch.zeros_like(ref_ds))
    assert torch.allclose(dscore.float(), ref_ds, atol=0.25, rtol=2e-2)
    ref_dr = dout.float().repeat_interleave(k, 0)[slots] * score.float()[slots][:, None]
    assert torch.allclose(drows[:n_valid].float(), ref_dr, atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_exp,k", [(16, 2), (4, 1), (64, 3), (200, 8)])
def test_gate_topk_softmax(dtype, n_exp, k):
    from fastmoe_b200.ops import gating
    torch.manual_seed(7)
    logits = torch.randn(500, n_exp, device=DEV, dtype=dtype).requires_grad_(True)
    idx, prob = gating.topk_softmax(logits, k)
    ref_l = logits.detach().float().requires_grad_(True)
    rv, _ri = torch.topk(ref_l, k, dim=-1)
    # Ties (frequent in bf16) may be ordered differently: compare the selected values, and
    # differentiate the reference through the kernel's own selection.
    picked = torch.gather(ref_l, 1, idx)
    assert torch.equal(picked.detach(), rv.detach())
    rp = torch.softmax(picked, -1)
    assert torch.allclose(prob.float(), rp, atol=1e-2 if dtype != torch.float32 else 1e-5)
    g = torch.randn_like(prob)
    prob.backward(g)
    rp.backward(g.float())
    assert torch.allclose(logits.grad.float(), ref_l.grad, atol=2e-2 if dtype != torch.float32 else 1e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("n_exp,k,d,bias", [(4, 2, 64, True), (16, 2, 1024, True), (13, 3, 200, False),
                                            (32, 1, 512, True), (64, 4, 256, True)])
def test_gate_linear_topk_softmax(dtype, n_exp, k, d, bias):
    r"""Single-pass linear gate against fp32 ``linear`` → ``topk`` → ``softmax``, forward and backward,
    with gradients arriving through the probabilities and through the logits."""
    from fastmoe_b200.ops import gating
    torch.manual_seed(11)
    n = 777
    x = torch.randn(n, d, device=DEV, dtype=dtype).requires_grad_(True)
    w = (torch.randn(n_exp, d, device=DEV) / d ** 0.5).to(dtype).requires_grad_(True)
    b = (torch.randn(n_exp, device=DEV) * 0.1).to(dtype).requires_grad_(True) if bias else None
    # the autograd function directly: the public wrapper only picks it for small expert counts
    logits, idx, prob = gating._LinearTopkSoftmax.apply(x, w, b, k)
    assert logits.dtype == dtype and idx.dtype == torch.int64 and prob.shape == (n, k)

    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    br = b.detach().float().requires_grad_(True) if bias else None
    lr = torch.nn.functional.linear(xr, wr, br)
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
    assert torch.allclose(logits.float(), lr, atol=tol, rtol=tol)
    # the selection is made on the rounded logits the kernel returns
    rv, _ = torch.topk(logits.detach().float(), k, dim=-1)
    assert torch.equal(torch.gather(logits.detach().float(), 1, idx), rv)
    rp = torch.softmax(torch.gather(lr, 1, idx), -1)
    assert torch.allclose(prob.float(), rp, atol=tol)

    gp = torch.randn_like(prob)
    gl = torch.randn_like(logits) * 0.1
    torch.autograd.backward([prob, logits], [gp, gl])
    torch.autograd.backward([rp, lr], [gp.float(), gl.float()])

    def close(a, r):
        scale = r.abs().max().item() + 1e-6
        return (a.float() - r).abs().max().item() <= 2e-2 * scale

    assert close(x.grad, xr.grad)
    assert close(w.grad, wr.grad)
    if bias:
        assert close(b.grad, br.grad)

    # gradient through the probabilities only (the plain top-k gate)
    x2 = x.detach().clone().requires_grad_(True)
    _, _, p2 = gating._LinearTopkSoftmax.apply(x2, w.detach(), None if b is None else b.detach(), k)
    p2.backward(gp)
    xr2 = x.detach().float().requires_grad_(True)
    lr2 = torch.nn.functional.linear(xr2, wr.detach(), None if br is None else br.detach())
    torch.softmax(torch.gather(lr2, 1, idx), -1).backward(gp.float())
    assert close(x2.grad, xr2.grad)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("n_exp,k,d,bias", [(16, 2, 1024, True), (64, 4, 512, True), (100, 8, 256, False),
                                            (256, 2, 1024, True)])
def test_gate_tensor_core_many_experts(dtype, n_exp, k, d, bias):
    r"""The linear gate above 8 experts: logits on the tcgen05 kernel (one group, expert
    dimension padded), top-k / softmax kernel, against fp32 ``linear`` -> ``topk`` -> ``softmax``,
    forward and backward through probabilities and logits."""
    from fastmoe_b200.ops import gating
    torch.manual_seed(12)
    n = 1531
    x = torch.randn(n, d, device=DEV, dtype=dtype).requires_grad_(True)
    w = (torch.randn(n_exp, d, device=DEV) / d ** 0.5).to(dtype).requires_grad_(True)
    b = (torch.randn(n_exp, device=DEV) * 0.1).to(dtype).requires_grad_(True) if bias else None
    assert gating._gate_gemm_ok(x, w, b)
    logits, idx, prob = gating.linear_topk_softmax(x, w, b, k)
    assert logits.shape == (n, n_exp) and idx.shape == (n, k) and int(idx.max()) < n_exp

    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    br = b.detach().float().requires_grad_(True) if bias else None
    lr = torch.nn.functional.linear(xr, wr, br)
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
    assert torch.allclose(logits.float(), lr, atol=tol, rtol=tol)
    rv, _ = torch.topk(logits.detach().float(), k, dim=-1)
    assert torch.equal(torch.gather(logits.detach().float(), 1, idx), rv)
    rp = torch.softmax(torch.gather(lr, 1, idx), -1)
    assert torch.allclose(prob.float(), rp, atol=tol)

    gp = torch.randn_like(prob)
    gl = torch.randn(n, n_exp, device=DEV, dtype=dtype) * 0.1
    torch.autograd.backward([prob, logits], [gp, gl])
    torch.autograd.backward([rp, lr], [gp.float(), gl.float()])
    for got, ref in ((x.grad, xr.grad), (w.grad, wr.grad)) + (((b.grad, br.grad),) if bias else ()):
        scale = ref.abs().max().item() + 1e-6
        assert (got.float() - ref).abs().max().item() <= 3e-2 * scale
    assert _native().read_status(0) == 0
