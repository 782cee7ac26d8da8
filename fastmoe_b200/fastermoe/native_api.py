r"""
The callback-driven entry points of the reference's native smart scheduler.

Parity: ``fmoe_cuda.smart_sch_forward`` / ``smart_sch_backward`` / ``reduce_grad``
(``cuda/fmoe_cuda.cpp:74-102,112-114``; implementation ``cuda/fastermoe/smart_schedule.h:
106-261,265-419`` and ``smart_schedule.cpp:41-63``).  Code written against the reference's
``MoEForward`` autograd function calls these three functions with Python callbacks that run
one expert on a buffer slice, fetch / stash / restore flat expert parameters and collect
gradients; the functions own the exchange schedule.

What is kept: the signatures, the callback contracts, the group-wise pipeline
(``FMOE_FASTER_GROUP_SIZE`` ranks per step, step ``s`` sends to group ``mine + s`` and receives
from group ``mine - s``), shadowed experts (parameter broadcast from the owner, local
evaluation on the rank's own rows, gradient reduction to the owner).  What differs: the
per-step plan comes from the native planner (``csrc/cpu/cpu_ops.cpp::smart_schedule_plan``), a
step's rows travel as one variable-size all-to-all instead of one send/recv pair per (expert,
peer), the parameter broadcast and the gradient reduction use the peer-to-peer kernels on
B200s, and all dispatch exchanges are queued on a side stream up front so that step ``s + 1``
is in flight while the experts work on step ``s``.

``store_idx`` handed to the callbacks: ``step * num_expert + e`` for the pipelined experts,
``world_size * num_expert + g`` for shadowed global expert ``g`` — unique per call, below
``2 * world_size * num_expert`` as the reference's callers assume.
"""
import torch
import torch.distributed as dist

from ..parallel.comm import get_moe_group
from .schedule import _comm_stream, _group_size, plan_steps


def _ctx(n_workers):
    group = get_moe_group() if n_workers > 1 else None
    me = dist.get_rank(group) if n_workers > 1 else 0
    return group, me


def _lists(lec, gec, stored):
    return ([int(v) for v in lec.reshape(-1).tolist()], [int(v) for v in gec.reshape(-1).tolist()],
            [bool(v) for v in stored.reshape(-1).tolist()])


def _all_to_all(buf, send_sizes, recv_sizes, group):
    out = buf.new_empty((sum(recv_sizes),) + tuple(buf.shape[1:]))
    if group is None:
        out.copy_(buf)
    else:
        dist.all_to_all_single(out, buf.contiguous(), recv_sizes, send_sizes, group=group)
    return out


def reduce_grad(t, root, expert_size):
    r"""Sum ``t[:expert_size]`` over the expert-parallel group into rank ``root`` (in place there)."""
    group = get_moe_group()
    if group is None or dist.get_world_size(group) == 1:
        return
    from ..parallel import symm
    flat = t.reshape(-1)[:expert_size]
    summed = symm.reduce_flat_to_owner(flat.contiguous(), int(root), group)
    if summed is not None:
        if dist.get_rank(group) == int(root):
            flat.copy_(summed)
        return
    buf = flat.contiguous().clone()
    dist.reduce(buf, dist.get_global_rank(group, int(root)), op=dist.ReduceOp.SUM, group=group)
    if dist.get_rank(group) == int(root):
        flat.copy_(buf)


class _Plan:
    r"""Everything both passes need to know about one call's schedule."""

    def __init__(self, lec, gec, stored_models, n_workers):
        self.world = int(n_workers)
        self.num_expert = lec.numel() // self.world
        self.group, self.me = _ctx(self.world)
        self.lec, self.gec, self.stored = _lists(lec, gec, stored_models)
        self.tot = self.num_expert * self.world
        self.gsz = _group_size(self.world)
        self.n_steps = self.world // self.gsz
        self.my_group = self.me // self.gsz
        (self.send_sizes, self.recv_sizes, self.send_ids,
         self.layouts) = plan_steps(lec, gec, stored_models, self.num_expert, self.world, self.me, self.gsz)
        self.seg = [0] * (self.tot + 1)
        for g in range(self.tot):
            self.seg[g + 1] = self.seg[g] + self.lec[g]

    def send_buffer(self, local_buf, step):
        pieces = [local_buf[self.seg[g]:self.seg[g + 1]] for g in self.send_ids[step]]
        return torch.cat(pieces) if pieces else local_buf[:0]

    def sources(self, step):
        from_group = (self.my_group - step) % self.n_steps
        return range(from_group * self.gsz, (from_group + 1) * self.gsz)

    def place_returned(self, out_buf, ret_buf, step):
        cursor = 0
        for g in self.send_ids[step]:
            n = self.lec[g]
            out_buf[self.seg[g]:self.seg[g + 1]] = ret_buf[cursor:cursor + n]
            cursor += n


def _pipeline(plan, local_buf, run_expert, width_out):
    r"""Exchange → per-expert callback → return exchange, for every step.  ``run_expert(x, y, e,
    store_idx)`` fills ``y``.  Returns ``(out_buf, list of received buffers)``."""
    dev = local_buf.device
    out_buf = local_buf.new_zeros((local_buf.shape[0], width_out))
    comm = _comm_stream(dev) if plan.group is not None else None
    main = torch.cuda.current_stream(dev) if comm is not None else None
    received, arrived = [], []
    if comm is not None:
        comm.wait_stream(main)
    for step in range(plan.n_steps):
        send = plan.send_buffer(local_buf, step)
        if comm is not None:
            with torch.cuda.stream(comm):
                got = _all_to_all(send, plan.send_sizes[step], plan.recv_sizes[step], plan.group)
                ev = torch.cuda.Event()
                ev.record(comm)
            send.record_stream(comm)
            got.record_stream(main)
        else:
            got, ev = _all_to_all(send, plan.send_sizes[step], plan.recv_sizes[step], plan.group), None
        received.append(got)
        arrived.append(ev)
    kept = []
    for step in range(plan.n_steps):
        if arrived[step] is not None:
            main.wait_event(arrived[step])
        recv = received[step]
        layout = plan.layouts[step]
        back = recv.new_zeros((recv.shape[0], width_out))
        for e in range(plan.num_expert):
            if plan.stored[plan.me * plan.num_expert + e]:
                continue
            srcs = [s for s in plan.sources(step) if layout[(s, e)][1] > 0]
            if not srcs:
                continue
            # the rows of one expert come from several sources: make them one contiguous block
            x_e = torch.cat([recv[layout[(s, e)][0]:layout[(s, e)][0] + layout[(s, e)][1]] for s in srcs])
            y_e = x_e.new_empty((x_e.shape[0], width_out))
            run_expert(x_e, y_e, e, step * plan.num_expert + e)
            cursor = 0
            for s in srcs:
                off, n = layout[(s, e)]
                back[off:off + n] = y_e[cursor:cursor + n]
                cursor += n
            kept.append(x_e)
        ret = _all_to_all(back, plan.recv_sizes[step], plan.send_sizes[step], plan.group)
        plan.place_returned(out_buf, ret, step)
    return out_buf, kept


def smart_sch_forward(input_buf, local_expert_count, global_expert_count, stored_models,
                      global_batch_size, expert_size, n_workers, forward_fn, get_param_fn,
                      stash_fn, pop_fn):
    r"""Returns ``(local_output_buf, global_input_buf)``; ``forward_fn(x, y, expert_idx, store_idx)``
    runs one local expert, ``get_param_fn(out, expert_idx)`` fills a flat parameter buffer,
    ``stash_fn(params, store_idx, expert_idx)`` installs broadcast parameters into local expert
    ``expert_idx`` and ``pop_fn(expert_idx)`` restores it."""
    plan = _Plan(local_expert_count, global_expert_count, stored_models, n_workers)
    d = input_buf.shape[1]
    out_buf, kept = _pipeline(plan, input_buf, forward_fn, d)
    for g in range(plan.tot):
        if not plan.stored[g]:
            continue
        owner, e = divmod(g, plan.num_expert)
        params = input_buf.new_zeros(int(expert_size))
        if owner == plan.me:
            get_param_fn(params, e)
        if plan.group is not None:
            from ..parallel import symm
            pushed = symm.broadcast_flat(params, owner, plan.group)
            if pushed is not None:
                params = pushed.contiguous()
            else:
                dist.broadcast(params, dist.get_global_rank(plan.group, owner), group=plan.group)
        store_idx = plan.tot + g
        stash_fn(params, store_idx, 0)
        x = input_buf[plan.seg[g]:plan.seg[g + 1]]
        y = out_buf[plan.seg[g]:plan.seg[g + 1]]
        forward_fn(x, y, 0, store_idx)
        pop_fn(0)
    gib = torch.cat(kept) if kept else input_buf[:0]
    return out_buf, gib


def smart_sch_backward(grad_out_buf, local_expert_count, global_expert_count, stored_models,
                       buf_batch_size, global_batch_size, n_workers, backward_fn, stash_fn, pop_fn,
                       collect_fn, set_grad_fn):
    r"""Returns ``grad_in_buf``; ``backward_fn(grad_y, grad_x, expert_idx, store_idx)`` back-propagates
    one expert call of the forward pass, ``stash_fn(store_idx, expert_idx)`` re-installs the
    shadow parameters, ``collect_fn(store_idx, root, expert_idx)`` gathers the gradients and
    reduces them to ``root`` (it calls :func:`reduce_grad`), ``set_grad_fn(store_idx, expert_idx)``
    adds them to the owner's expert."""
    plan = _Plan(local_expert_count, global_expert_count, stored_models, n_workers)
    d = grad_out_buf.shape[1]
    grad_in, _kept = _pipeline(plan, grad_out_buf, backward_fn, d)
    for g in range(plan.tot):
        if not plan.stored[g]:
            continue
        owner, e = divmod(g, plan.num_expert)
        store_idx = plan.tot + g
        stash_fn(store_idx, 0)
        gy = grad_out_buf[plan.seg[g]:plan.seg[g + 1]]
        gx = grad_in[plan.seg[g]:plan.seg[g + 1]]
        backward_fn(gy, gx, 0, store_idx)
        collect_fn(store_idx, owner, 0)
        pop_fn(0)
        if owner == plan.me:
            set_grad_fn(store_idx, e)
    return grad_in
