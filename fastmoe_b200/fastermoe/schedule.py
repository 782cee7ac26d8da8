r"""
The smart schedule of FasterMoE: group-wise pipelined exchange and shadow experts.

Parity: ``fmoe/fastermoe/schedule.py`` (``MoEForward`` ``:15-114``,
``_fmoe_general_global_forward`` ``:120-147``) and the native scheduler
``cuda/fastermoe/smart_schedule.h:105-419``.  Enabled by ``FMOE_FASTER_SCHEDULE_ENABLE``;
``FMOE_FASTER_GROUP_SIZE`` (default 4) ranks form a group, the all-to-all is split into
``world_size / group_size`` steps — in step ``s`` a rank sends to group ``(mine + s)`` and
receives from group ``(mine - s)`` — and the experts start on the rows of a step while the
next step's rows are still in flight (the exchange runs on a side stream).

Shadow experts (``FMOE_FASTER_SHADOW_ENABLE`` or an explicit ``stored_models`` mask): the
owner broadcasts the flat parameters of a shadowed expert, every rank runs that expert on its
own tokens, and the parameter gradients are reduced back to the owner.

Differences from the reference.  The whole schedule is assembled from differentiable pieces
(chunk all-to-all, parameter broadcast, local scatter/gather), so autograd derives the
backward schedule — reverse exchanges on the same side stream, gradient reduce-to-owner as the
backward of the broadcast — instead of a second hand-written native pass with Python
callbacks; bf16 therefore works in backward (the reference dispatches only fp32/fp64/fp16
there, ``cuda/fastermoe/smart_schedule.cpp:157``).  Shadowed experts are evaluated
functionally with the received parameters; local expert 0 is not overwritten and restored.
``FMoETransformerMLP`` without shadowing does not need this module on a GPU: its fused path
already overlaps the exchange with the expert GEMMs at row granularity.
"""
import torch
import torch.distributed as dist
from torch.autograd import Function

from .. import config
from ..functions import _local_gather, _local_scatter, prepare_forward
from ..parallel.comm import get_moe_group
from . import expert_utils
from .shadow_policy import get_shadow_policy, set_element_size

_comm_streams = {}


def _comm_stream(device):
    if device.type != "cuda":
        return None
    s = _comm_streams.get(device.index)
    if s is None:
        s = torch.cuda.Stream(device=device)
        _comm_streams[device.index] = s
    return s


class _ChunkAllToAll(Function):
    r"""``all_to_all_single`` with explicit split sizes; backward swaps the sizes."""

    @staticmethod
    def forward(ctx, buf, anchor, send_sizes, recv_sizes, group):
        # `anchor` is a zero-size leaf that requires grad: the output then requires grad on
        # every rank, so every rank runs this node's backward (a collective).
        ctx.sizes = (send_sizes, recv_sizes, group)
        out = buf.new_empty((sum(recv_sizes),) + tuple(buf.shape[1:]))
        dist.all_to_all_single(out, buf.contiguous(), recv_sizes, send_sizes, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        send_sizes, recv_sizes, group = ctx.sizes
        out = grad.new_empty((sum(send_sizes),) + tuple(grad.shape[1:]))
        dist.all_to_all_single(out, grad.contiguous(), send_sizes, recv_sizes, group=group)
        return out, None, None, None, None


class _BroadcastParams(Function):
    r"""Owner's flat parameters to every rank; backward sums the gradients at the owner.

    On B200s both directions are single peer-to-peer kernels: the owner pushes the parameters
    into every peer's symmetric buffer (one write per peer), and in backward the owner alone
    reads and sums the peers' gradient buffers.  Elsewhere: the collective library."""

    @staticmethod
    def forward(ctx, flat, anchor, owner_global_rank, is_owner, group):
        ctx.args = owner_global_rank, is_owner, group
        from ..parallel import symm
        owner_in_group = dist.get_group_rank(group, owner_global_rank) if group is not None \
            else owner_global_rank
        ctx.owner_in_group = owner_in_group
        pushed = symm.broadcast_flat(flat, owner_in_group, group)
        if pushed is not None:
            return pushed
        buf = flat.detach().clone()
        dist.broadcast(buf, owner_global_rank, group=group)
        return buf

    @staticmethod
    def backward(ctx, grad):
        owner, is_owner, group = ctx.args
        from ..parallel import symm
        summed = symm.reduce_flat_to_owner(grad.contiguous(), ctx.owner_in_group, group)
        if summed is not None:
            return summed, None, None, None, None
        grad = grad.contiguous().clone()
        dist.reduce(grad, owner, op=dist.ReduceOp.SUM, group=group)
        return (grad if is_owner else torch.zeros_like(grad)), None, None, None, None


class _Tie(Function):
    r"""Identity on ``main`` that also makes ``deps`` ancestors of the result.

    Every rank must run the backward of every collective, in the same order, even when it
    sent or received no rows in a step; tying zero-row slices of the collectives' outputs to
    the final result keeps those nodes in the autograd graph.
    """

    @staticmethod
    def forward(ctx, main, *deps):
        ctx.meta = [(d.shape, d.dtype, d.device) for d in deps]
        return main.view_as(main)

    @staticmethod
    def backward(ctx, grad):
        return (grad,) + tuple(torch.zeros(s, dtype=t, device=v) for s, t, v in ctx.meta)


def _run_shadow_expert(experts, flat, x):
    r"""Evaluate an expert of the layer's structure with parameters taken from ``flat``."""
    if isinstance(experts, (torch.nn.ModuleList, list, tuple)):
        module = experts[0]
        params, offset = {}, 0
        for name, p in module.named_parameters():
            params[name] = flat[offset:offset + p.numel()].view(p.shape)
            offset += p.numel()
        count = torch.tensor([x.shape[0]], dtype=torch.int64)
        return torch.func.functional_call(module, params, (x, count))
    w1, b1, w2, b2 = expert_utils.unflatten_like(experts, flat, 0)
    hid = experts.activation(torch.nn.functional.linear(x.type_as(w1), w1, b1))
    return torch.nn.functional.linear(hid, w2, b2)


def _group_size(world_size):
    g = min(config.faster_group_size(), world_size)
    while world_size % g != 0:
        g -= 1
    return max(g, 1)


def _plan_steps_python(lec_l, gec_l, stored, num_expert, world_size, me, gsz):
    r"""PyTorch-free restatement of the native chunk planner (same return layout, as lists)."""
    n_steps = world_size // gsz
    my_group = me // gsz
    send_sizes, recv_sizes, send_experts, recv_layout = [], [], [], []
    for step in range(n_steps):
        to_group = (my_group + step) % n_steps
        from_group = (my_group - step) % n_steps
        ss, rs, ids = [0] * world_size, [0] * world_size, []
        for p in range(to_group * gsz, (to_group + 1) * gsz):
            for e in range(num_expert):
                g = p * num_expert + e
                if not stored[g] and lec_l[g] > 0:
                    ids.append(g)
                    ss[p] += lec_l[g]
        layout, cursor = {}, 0
        for src in range(from_group * gsz, (from_group + 1) * gsz):
            for e in range(num_expert):
                if stored[me * num_expert + e]:
                    continue
                n = gec_l[src * num_expert + e]
                rs[src] += n
                layout[(src, e)] = (cursor, n)
                cursor += n
        send_sizes.append(ss)
        recv_sizes.append(rs)
        send_experts.append(ids)
        recv_layout.append(layout)
    return send_sizes, recv_sizes, send_experts, recv_layout


def plan_steps(lec, gec, stored_models, num_expert, world_size, me, gsz):
    r"""Per step of the group-wise exchange: split sizes, the expert segments that make up the
    send buffer, and where each (source rank, local expert) block sits in the received buffer.

    Computed by the native planner (``csrc/cpu/cpu_ops.cpp::smart_schedule_plan``, the
    counterpart of the pointer bookkeeping in ``cuda/fastermoe/smart_schedule.h:48-80``) when
    the extension is loaded, by :func:`_plan_steps_python` otherwise.
    """
    from ..ops import native
    if native.available():
        ss, rs, ids, offs, cur, cnt = native.get().cpu_smart_schedule_plan(
            lec.reshape(-1).cpu(), gec.reshape(-1).cpu(), stored_models.reshape(-1).cpu(),
            num_expert, world_size, me, gsz)
        n_steps = world_size // gsz
        my_group = me // gsz
        ids, offs = ids.tolist(), offs.tolist()
        cur, cnt = cur.tolist(), cnt.tolist()
        layouts = []
        for step in range(n_steps):
            from_group = (my_group - step) % n_steps
            layouts.append({(from_group * gsz + i, e): (cur[step][i][e], cnt[step][i][e])
                            for i in range(gsz) for e in range(num_expert) if cur[step][i][e] >= 0})
        return (ss.tolist(), rs.tolist(), [ids[offs[s]:offs[s + 1]] for s in range(n_steps)], layouts)
    stored = [bool(v) for v in stored_models.reshape(-1).tolist()]
    return _plan_steps_python([int(v) for v in lec.reshape(-1).tolist()],
                              [int(v) for v in gec.reshape(-1).tolist()], stored, num_expert,
                              world_size, me, gsz)


def smart_schedule_forward(expert_fn, experts, inp, pos_s, pos_g, lec, gec, stored_models,
                           fwd_batch_size, out_batch_size, num_expert, world_size):
    r"""Body of :class:`MoEForward`; all arguments as in the reference's ``MoEForward.forward``."""
    group = get_moe_group() if world_size > 1 else None
    me = dist.get_rank(group) if world_size > 1 else 0
    dev = inp.device
    stored = [bool(v) for v in stored_models.reshape(-1).tolist()]
    lec_l = [int(v) for v in lec.reshape(-1).tolist()]
    gec_l = [int(v) for v in gec.reshape(-1).tolist()]
    tot = num_expert * world_size

    local_input = _local_scatter(inp, pos_s)                 # rows grouped by global expert
    seg_start = [0] * (tot + 1)
    for g in range(tot):
        seg_start[g + 1] = seg_start[g] + lec_l[g]
    outputs = [None] * tot                                   # output rows per global expert segment
    ties = []                                                # zero-row slices of every exchanged buffer
    anchor = torch.zeros(0, device=dev, requires_grad=torch.is_grad_enabled())

    comm = _comm_stream(dev)
    main = torch.cuda.current_stream(dev) if comm is not None else None

    # ------------------------------------------------------------------ shadowed experts
    for g in range(tot):
        if not stored[g]:
            continue
        owner, e = divmod(g, num_expert)
        size = expert_utils.get_expert_param_size(experts, 0)
        if owner == me:
            flat = expert_utils.flat_expert_params(experts, e)
        else:
            ref = expert_utils.expert_parameters(experts, 0)[0]
            flat = torch.zeros(size, dtype=ref.dtype, device=ref.device)
        if world_size > 1:
            owner_global = dist.get_global_rank(group, owner) if group is not None else owner
            flat = _BroadcastParams.apply(flat, anchor, owner_global, owner == me, group)
        rows = local_input[seg_start[g]:seg_start[g + 1]]
        outputs[g] = _run_shadow_expert(experts, flat, rows)  # also with zero rows: keeps the graph uniform

    # ------------------------------------------------------------------ pipelined exchange
    # Three passes over the steps.  (1) All dispatch exchanges are queued on the side stream
    # at once, so the rows of step s + 1 travel while the experts work on step s.  (2) Per
    # step: wait for that step's rows, run the experts, queue the return exchange on the side
    # stream behind an event, and go on with the next step's experts while it travels.
    # (3) Collect the returned rows.  Every rank issues the collectives in the same order:
    # dispatch 0 .. n-1, return 0 .. n-1.
    gsz = _group_size(world_size)
    n_steps = world_size // gsz
    my_group = me // gsz
    all_send, all_recv, all_ids, all_layouts = plan_steps(lec, gec, stored_models, num_expert,
                                                         world_size, me, gsz)
    plans = []
    for step in range(n_steps):
        to_group = (my_group + step) % n_steps
        from_group = (my_group - step) % n_steps
        send_pieces = [local_input[seg_start[g]:seg_start[g + 1]] for g in all_ids[step]]
        send_buf = torch.cat(send_pieces) if send_pieces else local_input[:0]
        plans.append((to_group, from_group, send_buf, all_send[step], all_recv[step]))

    def exchange(buf, out_sizes, in_sizes, after=None):
        r"""One chunk all-to-all, on the side stream when there is one.  Returns the received
        buffer and the event that marks its arrival (None on the caller's stream)."""
        if comm is None:
            return _ChunkAllToAll.apply(buf, anchor, out_sizes, in_sizes, group), None
        if after is not None:
            comm.wait_event(after)
        with torch.cuda.stream(comm):
            got = _ChunkAllToAll.apply(buf, anchor, out_sizes, in_sizes, group)
            done = torch.cuda.Event()
            done.record(comm)
        buf.record_stream(comm)
        got.record_stream(main)
        return got, done

    received = []
    if world_size > 1:
        if comm is not None:
            comm.wait_stream(main)        # the send buffers were assembled on the caller's stream
        for _to, _from, send_buf, send_sizes, recv_sizes in plans:
            received.append(exchange(send_buf, send_sizes, recv_sizes))
    else:
        received = [(plan[2], None) for plan in plans]

    returned = []
    for step, (to_group, from_group, _send_buf, send_sizes, recv_sizes) in enumerate(plans):
        recv_buf, arrived = received[step]
        if arrived is not None:
            main.wait_event(arrived)
        if world_size > 1:
            ties.append(recv_buf[:0])

        # received layout: source rank outer, local expert inner
        pieces = all_layouts[step]
        result = {}
        for e in range(num_expert):
            if stored[me * num_expert + e]:
                continue
            srcs = [src for src in range(from_group * gsz, (from_group + 1) * gsz)
                    if pieces[(src, e)][1] > 0]
            if not srcs:
                continue
            x_e = torch.cat([recv_buf[pieces[(s, e)][0]:pieces[(s, e)][0] + pieces[(s, e)][1]]
                             for s in srcs])
            y_e = expert_fn(x_e, torch.tensor([x_e.shape[0]], dtype=torch.int64), e)
            cursor = 0
            for s in srcs:
                n = pieces[(s, e)][1]
                result[(s, e)] = y_e[cursor:cursor + n]
                cursor += n
        back = [result[(src, e)]
                for src in range(from_group * gsz, (from_group + 1) * gsz)
                for e in range(num_expert)
                if (src, e) in result]
        if back:
            back_buf = torch.cat(back)
        else:
            # nothing was computed here in this step, but peers may still expect the call
            back_buf = local_input.new_zeros((0, _feature_width(experts, local_input)))

        if world_size > 1:
            computed = None
            if comm is not None:
                computed = torch.cuda.Event()
                computed.record(main)
            returned.append(exchange(back_buf, recv_sizes, send_sizes, after=computed))
        else:
            returned.append((back_buf, None))

    for step, (to_group, _from, _send_buf, _send_sizes, _recv_sizes) in enumerate(plans):
        ret_buf, arrived = returned[step]
        if arrived is not None:
            main.wait_event(arrived)
        if world_size > 1:
            ties.append(ret_buf[:0])
        cursor = 0
        for p in range(to_group * gsz, (to_group + 1) * gsz):
            for e in range(num_expert):
                g = p * num_expert + e
                if not stored[g] and lec_l[g] > 0:
                    outputs[g] = ret_buf[cursor:cursor + lec_l[g]]
                    cursor += lec_l[g]

    kept = [o for o in outputs if o is not None and o.shape[0] > 0]
    if kept:
        local_output = torch.cat(kept)
    else:
        local_output = local_input.new_zeros((0, _feature_width(experts, local_input)))
    if ties:
        local_output = _Tie.apply(local_output, *ties)
    return _local_gather(local_output, pos_g, out_batch_size, maybe_overlap=False)


def _feature_width(experts, local_input):
    return local_input.shape[-1]


class MoEForward:
    r"""Call-compatible stand-in of the reference's autograd function: ``MoEForward.apply(...)``."""

    @staticmethod
    def apply(expert_fn, experts, inp, pos_s, pos_g, local_expert_count, global_expert_count,
              stored_models, fwd_batch_size, out_batch_size, num_expert, world_size):
        return smart_schedule_forward(expert_fn, experts, inp, pos_s, pos_g, local_expert_count,
                                      global_expert_count, stored_models, fwd_batch_size,
                                      out_batch_size, num_expert, world_size)


policy_fn = None


def _fmoe_general_global_forward(inp, gate, expert_fn, n_expert, world_size, experts=None,
                                 stored_models=None):
    r"""Smart-schedule replacement of the general forward (single tensor input only)."""
    assert isinstance(inp, torch.Tensor), "the smart schedule takes a single tensor input"
    pos, lec, gec, _fwd_expert_count, fwd_batch_size = prepare_forward(gate, n_expert, world_size)

    global policy_fn
    if policy_fn is None:
        policy_fn = get_shadow_policy(d_model=inp.shape[-1])
    set_element_size(inp.element_size())
    if stored_models is None:
        stored_models = policy_fn(lec, gec, n_expert, world_size, inp.device)

    topk = gate.shape[1] if gate.dim() == 2 else 1
    out_batch_size = inp.shape[0] * topk
    return MoEForward.apply(expert_fn, experts, inp,
                            torch.div(pos, topk, rounding_mode="floor"), pos, lec, gec,
                            stored_models, fwd_batch_size, out_batch_size, n_expert, world_size)
