r"""The C++ CPU ops of the extension against their PyTorch restatements (`ops/torch_impl.py`),
on randomly generated routing tables: both are oracles for the CUDA kernels, so they have to
agree with each other first.  Skipped when the extension has not been built."""
import pytest
import torch
from hypothesis import given, settings, strategies as st

from fastmoe_b200.ops import native, torch_impl

pytestmark = pytest.mark.skipif(not native.available(), reason="native extension not built")


def _routing(draw, tot):
    n = draw(st.integers(min_value=0, max_value=60))
    ids = draw(st.lists(st.integers(min_value=-1, max_value=tot - 1), min_size=n, max_size=n))
    return torch.tensor(ids, dtype=torch.int64)


@st.composite
def routing_case(draw):
    n_expert = draw(st.integers(min_value=1, max_value=5))
    n_worker = draw(st.integers(min_value=1, max_value=4))
    return n_expert, n_worker, _routing(draw, n_expert * n_worker)


@settings(max_examples=60, deadline=None, derandomize=True)
@given(routing_case())
def test_route_matches_restatement(case):
    n_expert, n_worker, idx = case
    tot = n_expert * n_worker
    counts, rank = native.get().cpu_route(idx, tot)
    assert torch.equal(counts.long(), torch_impl.expert_count(idx, tot).long())
    assert torch.equal(rank.long(), torch_impl.slot_rank(idx, tot).reshape(-1).long())
    # the positions implied by (count prefix, rank) are a permutation of the kept slots
    pos = torch_impl.assign_pos(idx, tot)
    assert sorted(pos.tolist()) == [s for s, e in enumerate(idx.tolist()) if e >= 0]
    assert idx[pos].tolist() == sorted(e for e in idx.tolist() if e >= 0)


@settings(max_examples=60, deadline=None, derandomize=True)
@given(routing_case(), st.integers(min_value=0, max_value=12))
def test_capacity_limit_and_prune_match_restatement(case, capacity):
    n_expert, n_worker, idx = case
    tot = n_expert * n_worker
    gen = torch.Generator().manual_seed(int(idx.sum()) % 1000 + capacity)
    proposals = torch.randint(0, 9, (tot,), generator=gen)
    cap_a = torch.full((n_expert,), capacity, dtype=torch.int32)
    cap_b = cap_a.clone()
    got = native.get().cpu_limit_by_capacity(proposals.clone(), cap_a, n_expert, n_worker)
    want = torch_impl.limit_by_capacity(proposals.clone(), cap_b, n_expert, n_worker)
    assert torch.equal(got, want) and torch.equal(cap_a, cap_b)
    # grants never exceed the capacity of an expert and are handed out in worker order
    per_expert = got.view(n_worker, n_expert)
    assert bool((per_expert.sum(0) <= capacity).all())
    budget = torch.randint(0, 6, (tot,), generator=gen).to(torch.int32)
    budget_a, budget_b = budget.clone(), budget.clone()
    pruned = native.get().cpu_prune_gate_by_capacity(idx.clone(), budget_a, n_expert, n_worker)
    ref = torch_impl.prune_gate_by_capacity(idx.clone(), budget_b, n_expert, n_worker)
    assert torch.equal(pruned, ref)
    # an expert keeps at most what it was asked for and at most its budget
    kept = torch_impl.expert_count(pruned, tot).long()
    assert bool((kept <= torch_impl.expert_count(idx, tot).long()).all())
    assert bool((kept <= budget.long()).all())


@settings(max_examples=40, deadline=None, derandomize=True)
@given(st.integers(min_value=1, max_value=5), st.integers(min_value=0, max_value=10_000))
def test_swipe_plan_matches_restatement_and_conserves_tokens(n_worker, seed):
    gen = torch.Generator().manual_seed(seed)
    want = torch.randint(0, 20, (n_worker, n_worker), generator=gen)
    cap = torch.randint(0, 40, (n_worker,), generator=gen)
    accepted, left = native.get().cpu_swipe_plan(want, cap)
    ref_accepted, ref_left = torch_impl.swipe_plan(want.tolist(), cap.tolist(), n_worker)
    assert accepted.tolist() == ref_accepted and left.tolist() == ref_left
    # nobody receives more than its capacity; tokens are only lost when all capacity is used up
    assert bool((accepted.sum(0) <= cap).all())
    lost = int(want.sum()) - int(accepted.sum())
    assert lost >= 0 and (lost == 0 or int(left.sum()) == 0)


@settings(max_examples=25, deadline=None, derandomize=True)
@given(st.integers(min_value=1, max_value=4), st.integers(min_value=0, max_value=1000))
def test_grouped_linear_matches_restatement(n_expert, seed):
    gen = torch.Generator().manual_seed(seed)
    counts = torch.randint(0, 6, (n_expert,), generator=gen)
    rows, d_in, d_out = int(counts.sum()), 5, 3
    x = torch.randn(rows, d_in, generator=gen, dtype=torch.float64)
    w = torch.randn(n_expert, d_out, d_in, generator=gen, dtype=torch.float64)
    b = torch.randn(n_expert, d_out, generator=gen, dtype=torch.float64)
    nat = native.get()
    y = nat.cpu_linear_forward(x, counts, w, b)
    assert torch.allclose(y, torch_impl.linear_forward(x, counts, w, b))
    gy = torch.randn(rows, d_out, generator=gen, dtype=torch.float64)
    gx, gw, gb = nat.cpu_linear_backward(gy, x, counts, w, b)
    rx, rw, rb = torch_impl.linear_backward(gy, x, counts, w, b)
    assert torch.allclose(gx, rx) and torch.allclose(gw, rw) and torch.allclose(gb, rb)


@settings(max_examples=50, deadline=None, derandomize=True)
@given(st.integers(min_value=1, max_value=8), st.integers(min_value=1, max_value=4),
       st.integers(min_value=0, max_value=10_000))
def test_exchange_offsets_tile_every_receive_buffer_exactly(world, n_expert, seed):
    r"""The offsets every rank derives from the shared count matrix are consistent: on each
    receiving rank the row ranges of all (source, expert) pairs are disjoint, ordered by local
    expert then source position (own rows first), and cover ``[0, total)``; grants obey the
    capacities and equal the two-step exchange of the collective-library path."""
    gen = torch.Generator().manual_seed(seed)
    tot = world * n_expert
    mat = torch.randint(0, 7, (world, tot), generator=gen)
    views = [torch_impl.exchange_offsets(mat, me, n_expert) for me in range(world)]
    for owner in range(world):
        _base, offs, total, overflow = views[owner]
        assert not overflow and total == int(mat[:, owner * n_expert:(owner + 1) * n_expert].sum())
        covered = []
        for e in range(n_expert):
            g = owner * n_expert + e
            for src in range(world):
                start = int(views[src][0][g])
                n = int(mat[src, g])
                assert int(offs[e]) <= start and start + n <= int(offs[e + 1])
                covered.append((start, start + n))
            # inside the segment: own rows first, then the rows of rank owner - 1, owner - 2, ...
            by_pos = [int(views[(owner - j) % world][0][g]) for j in range(world)]
            assert by_pos == sorted(by_pos) and by_pos[0] == int(offs[e])
        covered = [c for c in covered if c[1] > c[0]]
        covered.sort()
        assert all(a[1] == b[0] for a, b in zip(covered, covered[1:]))
        if covered:
            assert covered[0][0] == 0 and covered[-1][1] == total
    # the walk order of the row blocks: every block once, source position of the last row never
    # decreasing; and the senders' item lists cover, per owner, every (block, source) pair that
    # the owner's arrival flags wait for
    block = 4
    for owner in range(world):
        _base, offs, total, _ov = views[owner]
        order = torch_impl.exchange_block_order(mat, owner, n_expert, block=block)
        want = [(e, m) for e in range(n_expert)
                for m in range((int(offs[e + 1]) - int(offs[e]) + block - 1) // block)]
        assert sorted(order) == want
        stages = []
        for e, m in order:
            last = min(int(offs[e]) + (m + 1) * block, int(offs[e + 1])) - 1
            g = owner * n_expert + e
            pos = [j for j in range(world)
                   if int(views[(owner - j) % world][0][g]) <= last
                   < int(views[(owner - j) % world][0][g]) + int(mat[(owner - j) % world, g])]
            assert len(pos) == 1
            stages.append(pos[0])
        assert stages == sorted(stages)
    for me in range(world):
        prefix = torch_impl.send_item_prefix(mat, me, n_expert, block=block)
        assert len(prefix) == tot + 1 and prefix[0] == 0
        for j in range(world):
            owner = (me + j) % world
            for e in range(n_expert):
                g = owner * n_expert + e
                start, n = int(views[me][0][g]) - int(views[owner][1][e]), int(mat[me, g])
                touched = len({r // block for r in range(start, start + n)})
                assert prefix[j * n_expert + e + 1] - prefix[j * n_expert + e] == touched
    # the senders' items against what the owners' tiles wait for: tile (expert e, block m) of
    # owner p waits for the flag (blk_base + m, source w) of every source whose rows overlap the
    # block; exactly those flags must be raised, each by one item that carries exactly the
    # overlapping rows — also when the buffers are too small and rows are dropped
    for cap in (None, max(1, int(mat.sum()) // (2 * world))):
        raised = {}
        for me in range(world):
            items = torch_impl.send_items(mat, me, n_expert, cap, block=block)
            prefix = torch_impl.send_item_prefix(mat, me, n_expert, cap, block=block)
            assert len(items) == prefix[-1]
            for owner, flag_blk, r0, r1 in items:
                assert (owner, flag_blk, me) not in raised and r0 < r1
                raised[(owner, flag_blk, me)] = (r0, r1)
        waited = {}
        for owner in range(world):
            _b, offs, _t, _o = torch_impl.exchange_offsets(mat, owner, n_expert, cap)
            limit = int(offs[-1])
            blk0 = 0
            for e in range(n_expert):
                g = owner * n_expert + e
                lo, hi = int(offs[e]), int(offs[e + 1])
                for m in range((hi - lo + block - 1) // block):
                    r0, r1 = lo + m * block, min(lo + (m + 1) * block, hi)
                    for w in range(world):
                        s0 = int(views[w][0][g])
                        s1 = min(s0 + int(mat[w, g]), limit)
                        # the producer's test (grouped_gemm_kernel.cuh, gate_flag): a source
                        # with rows of its own that overlap the block
                        if s0 < s1 and s0 < r1 and s1 > r0:
                            waited[(owner, blk0 + m, w)] = (max(s0, r0), min(s1, r1))
                # flag blocks are numbered over the unclamped segments (what the senders know)
                blk0 += (int(mat[:, g].sum()) + block - 1) // block
        assert raised == waited
    # a bounded receive buffer: totals are clamped and the overflow is flagged on every rank
    small = max(0, int(mat.sum()) // (2 * world))
    flags = [torch_impl.exchange_offsets(mat, me, n_expert, small)[3] for me in range(world)]
    assert len(set(flags)) == 1
    caps = torch.randint(0, 12, (world, n_expert), generator=gen)
    grant = torch_impl.capacity_grants(mat, caps, n_expert)
    for owner in range(world):
        cap = caps[owner].to(torch.int32).clone()
        proposals = mat[:, owner * n_expert:(owner + 1) * n_expert].reshape(-1).clone()
        two_step = torch_impl.limit_by_capacity(proposals, cap, n_expert, world).view(world, n_expert)
        assert torch.equal(grant[:, owner * n_expert:(owner + 1) * n_expert], two_step)
        assert bool((two_step.sum(0) <= caps[owner]).all())
