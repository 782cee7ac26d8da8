r"""
Plain-PyTorch restatement of every native op.

Three uses: (1) execution path for CPU tensors when the extension is not built,
(2) fp32 oracle that the sm_100a kernels are tested against, (3) fallback for dtypes the
tensor-core kernels do not cover (fp64).  Semantics follow the reference's native entry
points (``cuda/fmoe_cuda.cpp:17-102``) with one deliberate difference: wherever the
reference lets atomics decide an order (``cuda/local_exchange.cuh:5-16``,
``cuda/balancing.cuh:5-45``) the order here is fixed — slots are ranked by their index,
workers by their rank — so results are reproducible.
"""
import torch


# ----------------------------------------------------------------------------------
# Routing bookkeeping
# ----------------------------------------------------------------------------------
def expert_count(gate_idx, tot_expert):
    r"""Histogram of routing ids over ``tot_expert`` bins; ``-1`` (dropped) is skipped.

    Parity: ``cuda/local_exchange.cuh:36-69``.
    """
    flat = gate_idx.reshape(-1)
    valid = flat[flat >= 0]
    return torch.bincount(valid, minlength=tot_expert)[:tot_expert].to(torch.int32)


def assign_pos(gate_idx, tot_expert):
    r"""Slot ids grouped by ascending expert, ascending slot id inside an expert.

    Parity: ``cuda/local_exchange.cuh:5-26`` (there the inner order is whatever the
    atomics produce).  Returns ``pos`` of length ``sum(count)``.
    """
    flat = gate_idx.reshape(-1)
    key = torch.where(flat >= 0, flat, torch.full_like(flat, tot_expert))
    order = torch.sort(key, stable=True).indices
    n_valid = int((flat >= 0).sum())
    return order[:n_valid]


def slot_rank(gate_idx, tot_expert):
    r"""For every slot its 0-based rank among the slots routed to the same expert (``-1`` if dropped)."""
    flat = gate_idx.reshape(-1)
    out = torch.full_like(flat, -1)
    key = torch.where(flat >= 0, flat, torch.full_like(flat, tot_expert))
    sorted_key, order = torch.sort(key, stable=True)
    counts = torch.bincount(sorted_key, minlength=tot_expert + 1)
    starts = torch.cumsum(counts, 0) - counts
    rank_sorted = torch.arange(flat.numel(), device=flat.device) - starts[sorted_key]
    out[order] = rank_sorted
    out[flat < 0] = -1
    return out.view_as(gate_idx)


def limit_by_capacity(expert_count_w, capacity, n_expert, n_worker):
    r"""Grant capacity of each local expert to the workers in rank order.

    ``expert_count_w[w*E+e]`` is what worker ``w`` proposes for local expert ``e``;
    returns the granted counts with the same layout and decrements ``capacity`` in place
    by the proposals, like ``cuda/balancing.cuh:5-21`` does.
    """
    ec = expert_count_w.view(n_worker, n_expert).to(torch.int64)
    cap = capacity.to(torch.int64).view(1, n_expert)
    before = torch.cumsum(ec, 0) - ec
    left = (cap - before).clamp(min=0)
    grant = torch.minimum(ec, left)
    capacity.sub_(ec.sum(0).to(capacity.dtype))
    return grant.reshape(-1).to(expert_count_w.dtype)


def prune_gate_by_capacity(gate_idx, expert_count_cap, n_expert, n_worker):
    r"""Keep the first ``expert_count_cap[g]`` slots of every expert (slot order), drop the rest.

    Parity: ``cuda/balancing.cuh:32-45``; unlike it, ``-1`` inputs are passed through
    instead of indexing out of range.  ``expert_count_cap`` is decremented in place by the
    number of requests, as the reference's atomic does.
    """
    tot = n_expert * n_worker
    rank = slot_rank(gate_idx, tot)
    flat = gate_idx.reshape(-1)
    safe = flat.clamp(min=0)
    allowed = expert_count_cap.to(torch.int64)[safe]
    keep = (flat >= 0) & (rank.reshape(-1) < allowed)
    new_idx = torch.where(keep, flat, torch.full_like(flat, -1)).view_as(gate_idx)
    expert_count_cap.sub_(expert_count(gate_idx, tot).to(expert_count_cap.dtype))
    return new_idx


# ----------------------------------------------------------------------------------
# Grouped linear
# ----------------------------------------------------------------------------------
def _segments(counts):
    counts = [int(c) for c in counts.reshape(-1).tolist()]
    base = 0
    for e, n in enumerate(counts):
        yield e, base, base + n
        base += n


def linear_forward(inp, expert_count_cpu, weight, bias=None):
    r"""``out[rows_e] = inp[rows_e] @ weight[e].T + bias[e]`` (``cuda/parallel_linear.cuh:56-89``)."""
    out = inp.new_empty(inp.shape[0], weight.shape[1])
    for e, lo, hi in _segments(expert_count_cpu):
        if hi > lo:
            y = inp[lo:hi] @ weight[e].t()
            if bias is not None:
                y = y + bias[e]
            out[lo:hi] = y
    return out


def linear_backward(grad_out, inp, expert_count_cpu, weight, bias=None):
    r"""Input, weight and bias gradients of :func:`linear_forward` (``cuda/parallel_linear.cuh:92-163``).

    Experts that received no rows get zero weight/bias gradients.
    """
    grad_in = grad_out.new_empty(inp.shape[0], weight.shape[2])
    grad_w = torch.zeros_like(weight)
    grad_b = torch.zeros_like(bias) if bias is not None else None
    for e, lo, hi in _segments(expert_count_cpu):
        if hi > lo:
            grad_in[lo:hi] = grad_out[lo:hi] @ weight[e]
            grad_w[e] = grad_out[lo:hi].t() @ inp[lo:hi]
            if grad_b is not None:
                grad_b[e] = grad_out[lo:hi].sum(0)
    return grad_in, grad_w, grad_b


# ----------------------------------------------------------------------------------
# SWIPE re-balancing (single round), host algorithm on gathered counts
# ----------------------------------------------------------------------------------
def swipe_plan(counts_to_worker, capacity_left, n_worker):
    r"""Pure function at the heart of ``swipe_once`` (``cuda/balancing.cu:83-186``).

    ``counts_to_worker[i][j]``: tokens rank ``i`` wants to send to worker ``j``;
    ``capacity_left[j]``: what worker ``j`` can still accept.  Each worker accepts
    requests in rank order until it is full; the overflow of rank 0, 1, … is re-assigned
    greedily to the workers with spare capacity in rank order.  Returns the matrix of
    accepted counts ``new[i][j]`` and the remaining capacity per worker.
    """
    want = [list(map(int, row)) for row in counts_to_worker]
    cap = [int(c) for c in capacity_left]
    accepted = [[0] * n_worker for _ in range(n_worker)]
    dropped = [0] * n_worker
    for j in range(n_worker):
        for i in range(n_worker):
            take = min(want[i][j], cap[j])
            accepted[i][j] = take
            cap[j] -= take
            dropped[i] += want[i][j] - take
    j = 0
    for i in range(n_worker):
        while dropped[i] > 0 and j < n_worker:
            take = min(dropped[i], cap[j])
            accepted[i][j] += take
            cap[j] -= take
            dropped[i] -= take
            if cap[j] == 0:
                j += 1
    return accepted, cap


def swipe_reassign(gate_idx, accepted_row, n_expert, bias):
    r"""Rewrite one rank's routing so that worker ``j`` gets exactly ``accepted_row[j]`` tokens.

    Tokens keep their expert while their worker still has room (slot order); the others go
    to expert ``bias`` of the first worker with room left.
    """
    idx = gate_idx.reshape(-1).clone()
    n_worker = len(accepted_row)
    worker = torch.div(idx, n_expert, rounding_mode="floor")
    quota = torch.tensor(accepted_row, dtype=torch.int64, device=idx.device)
    rank = slot_rank(worker, n_worker).reshape(-1)
    keep = rank < quota[worker.clamp(min=0)]
    kept_per_worker = torch.bincount(worker[keep], minlength=n_worker)[:n_worker]
    spare = (quota - kept_per_worker).clamp(min=0)
    moved = (~keep).nonzero().reshape(-1)
    if moved.numel() > 0:
        targets = torch.repeat_interleave(
            torch.arange(n_worker, device=idx.device), spare)[:moved.numel()]
        if targets.numel() < moved.numel():
            pad = torch.full((moved.numel() - targets.numel(),), -1,
                             dtype=torch.int64, device=idx.device)
            new_ids = torch.cat([targets * n_expert + bias, pad])
        else:
            new_ids = targets * n_expert + bias
        idx[moved] = new_ids
    return idx.view_as(gate_idx)


# ----------------------------------------------------------------------------------
# Expert-parallel exchange bookkeeping (restatement of the device-side arithmetic)
# ----------------------------------------------------------------------------------
def exchange_offsets(count_matrix, me, n_expert, capacity_rows=None):
    r"""What ``count_exchange_kernel`` derives on rank ``me`` from the full count matrix.

    ``count_matrix[w, g]``: slots rank ``w`` routes to global expert ``g`` (``g = owner * E + e``).
    Receive layout on every rank: local expert outer; inside an expert's segment the rows of
    source rank ``w`` sit at position ``(owner - w) mod world`` — the owner's own rows first, then
    those of rank ``owner - 1``, ``owner - 2``, ...  Returns

    * ``dst_base[g]``: row in the owner's receive buffer where this rank's rows for ``g`` start,
    * ``expert_offs[e]`` (``E + 1`` entries): row ranges of this rank's local experts,
    * ``total``: rows this rank receives (clamped to ``capacity_rows`` when given),
    * ``overflow``: whether any rank receives more than ``capacity_rows``.
    """
    mat = torch.as_tensor(count_matrix, dtype=torch.int64)
    world, tot = mat.shape
    assert tot == world * n_expert
    col = mat.sum(0)
    dst_base = torch.zeros(tot, dtype=torch.int64)
    for g in range(tot):
        owner, e = divmod(g, n_expert)
        before = sum(int(mat[(owner - j) % world, g]) for j in range((owner - me) % world))
        dst_base[g] = col[owner * n_expert:owner * n_expert + e].sum() + before
    mine = col[me * n_expert:(me + 1) * n_expert]
    expert_offs = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(mine, 0)])
    per_rank = col.view(world, n_expert).sum(1)
    overflow = capacity_rows is not None and bool((per_rank > capacity_rows).any())
    if capacity_rows is not None:
        expert_offs = expert_offs.clamp(max=capacity_rows)
    return dst_base, expert_offs, int(expert_offs[-1]), overflow


def exchange_block_order(count_matrix, me, n_expert, capacity_rows=None, block=128):
    r"""The order in which rank ``me`` walks the ``block``-row blocks of its receive buffer
    (``count_exchange_kernel``'s ``blk_order``): by the source position of a block's last row —
    own rows first, then the rows of rank ``me - 1``, ... — then local expert, then row.  Blocks
    of expert ``e`` whose last row comes from position ``j`` are consecutive: with ``f(t)`` the
    number of blocks whose last row lies below row ``t`` of the segment they are
    ``[f(s_j), f(s_{j+1}))``, ``s_j`` being where position ``j`` starts.  Returns a list of
    ``(local expert, block inside the expert)``."""
    mat = torch.as_tensor(count_matrix, dtype=torch.int64)
    world = mat.shape[0]
    cap = capacity_rows if capacity_rows is not None else int(mat.sum())
    starts = []          # starts[e][j]: row where position j of expert e begins, clamped
    run = 0
    for e in range(n_expert):
        row = []
        for j in range(world + 1):
            row.append(min(run, cap))
            if j < world:
                run += int(mat[(me - j) % world, me * n_expert + e])
        starts.append(row)
    order = []
    for j in range(world):
        for e in range(n_expert):
            n_e = starts[e][world] - starts[e][0]
            n_blk = (n_e + block - 1) // block

            def below(t, n_e=n_e, n_blk=n_blk):
                return n_blk if t >= n_e else t // block
            lo = below(starts[e][j] - starts[e][0])
            hi = below(starts[e][j + 1] - starts[e][0])
            order.extend((e, m) for m in range(lo, hi))
    return order


def send_item_prefix(count_matrix, me, n_expert, capacity_rows=None, block=128):
    r"""``item_prefix`` of ``count_exchange_kernel``: exclusive prefix of the number of
    ``block``-row blocks of the owner's buffer that this rank's rows touch, per (peer distance
    ``j``, local expert ``e``) pair in send order — ``j`` outer, ``e`` inner, global expert
    ``((me + j) mod world) * E + e``."""
    mat = torch.as_tensor(count_matrix, dtype=torch.int64)
    world = mat.shape[0]
    cap = capacity_rows if capacity_rows is not None else int(mat.sum())
    col = mat.sum(0)
    prefix = [0]
    for j in range(world):
        owner = (me + j) % world
        for e in range(n_expert):
            g = owner * n_expert + e
            seg = int(col[owner * n_expert:owner * n_expert + e].sum())
            before = sum(int(mat[(owner - i) % world, g]) for i in range((owner - me) % world))
            n = int(mat[me, g])
            end = min(before + n, cap - seg)
            items = 0
            if n > 0 and end > before:
                items = (end - 1) // block - before // block + 1
            prefix.append(prefix[-1] + items)
    return prefix


def send_items(count_matrix, me, n_expert, capacity_rows=None, block=128):
    r"""The sender warps' work list on rank ``me`` (``grouped_gemm_kernel.cuh::send_decode``): one
    item per ``block``-row block of an owner's buffer that this rank's rows touch, in send
    order.  Each item is ``(owner, flag block on the owner, first row, one past the last row)``
    with rows counted from the start of the owner's buffer; the owner's arrival flag
    ``(flag block, source = me)`` goes up when all rows of the item have been stored."""
    mat = torch.as_tensor(count_matrix, dtype=torch.int64)
    world = mat.shape[0]
    cap = capacity_rows if capacity_rows is not None else int(mat.sum())
    col = mat.sum(0)
    items = []
    for j in range(world):
        owner = (me + j) % world
        for e in range(n_expert):
            g = owner * n_expert + e
            seg = int(col[owner * n_expert:owner * n_expert + e].sum())
            blk_base = sum((int(col[owner * n_expert + e2]) + block - 1) // block for e2 in range(e))
            rel0 = sum(int(mat[(owner - i) % world, g]) for i in range((owner - me) % world))
            n = int(mat[me, g])
            end = min(rel0 + n, cap - seg)
            if n == 0 or end <= rel0:
                continue
            for b in range(rel0 // block, (end - 1) // block + 1):
                items.append((owner, blk_base + b, seg + max(rel0, b * block), seg + min(end, (b + 1) * block)))
    return items


def capacity_grants(count_matrix, capacities, n_expert):
    r"""What ``capacity_grant_kernel`` derives on every rank: ``grant[w, g]``, handed out in rank
    order from the capacity of ``g``'s owner (``capacities[owner, e]``)."""
    mat = torch.as_tensor(count_matrix, dtype=torch.int64)
    caps = torch.as_tensor(capacities, dtype=torch.int64)
    world, tot = mat.shape
    grant = torch.zeros_like(mat)
    for g in range(tot):
        owner, e = divmod(g, n_expert)
        left = int(caps[owner, e])
        for w in range(world):
            take = min(int(mat[w, g]), max(left, 0))
            grant[w, g] = take
            left -= take
    return grant
