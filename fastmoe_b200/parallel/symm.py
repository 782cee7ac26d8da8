r"""
Symmetric-memory workspace and the fused expert-parallel path on top of it.

Every rank of an expert-parallel group allocates the same staging buffers with
``torch.distributed._symmetric_memory`` (CUDA virtual-memory handles exchanged through the
group's store) and learns the peers' addresses.  The kernels of ``csrc/sm100/p2p.cu`` then
move token rows with NVLink stores and publish completion through flag words, which replaces
what the reference does with a private NCCL communicator obtained by subclassing
``ProcessGroupNCCL`` (``cuda/global_exchange.cpp:108-158``) and host loops of send/recv
(``cuda/global_exchange.h:28-53,73-98``).

One layer call is, per rank and without any host read:

    route → count_exchange (counts to all peers; offsets and block tables from the full matrix)
          → grouped GEMM 1 launch.  Two warps of every CTA that are idle in the GEMM roles are
            *senders*: they copy this rank's token rows (+ (source, slot) words) through
            registers into the owners' receive buffers and raise one arrival flag per (128-row
            block, source).  The GEMM roles of the same CTAs work (+ bias, activation) straight
            out of the receive buffer, tiles walked in the arrival order of their row blocks and
            every tile waiting only for the flags of its own block: dispatch and GEMM 1 overlap
            tile by tile
          → grouped GEMM 2 whose epilogue stores every output row straight into its source
            rank's slot-indexed return buffer and raises the return flags
          → wait_combine  (arrival flags, gate-weighted sum over the k slots of a token)

Backward runs the same two exchanges with gradient rows: the score-scaled output gradients
are sent by the sender warps of the first input-gradient GEMM, the last input-gradient GEMM
pushes from its epilogue.  Layers whose activation the GEMM epilogue does not know use the
stand-alone dispatch / return kernels around PyTorch ops.  The module also holds the other
peer-to-peer collectives: gradient all-reduce (one- and two-shot), all-gather of slice
groups, capacity grants.

Buffers.  The receive buffer of a layer call (rows kept for the weight gradient) is leased
from a pool of symmetric allocations and handed back when the backward pass is done; the
return buffer, the gradient receive buffer and the flag words are shared by all layers: a
rank can only start the next exchange after it has seen every peer's flags of the current one,
and a peer only raises them after it is done reading, so no buffer is overwritten early.
All of them are sized from ONE token budget per group, agreed once (see ``token_budget``);
ranks may bring different numbers of tokens as long as none exceeds the budget.

Requirements of the fused path: one process per GPU on one NVLink domain, at most 16 ranks.
"""
import math
import os

import torch
import torch.distributed as dist
from torch.autograd import Function

from .. import config
from ..ops import native
from ..utils.profiling import fused_range, new_ep_trace

_WORKSPACES = {}
_FAILED = set()
_MAX_TOT_EXPERT = 4096


def _group_key(group, device):
    name = getattr(group, "group_name", None) or str(id(group))
    return (name, device.index)


class SymmWorkspace:
    r"""Symmetric buffers, peer address tables and the native exchange context of one group."""

    def __init__(self, group, device):
        import torch.distributed._symmetric_memory as symm_mem
        self._symm_mem = symm_mem
        self.group = group
        self.device = device
        self.world = dist.get_world_size(group)
        self.me = dist.get_rank(group)
        nat = native.get()
        if self.world > nat.P2P_MAX_PEERS:
            raise RuntimeError("fused expert parallelism supports at most %d ranks" % nat.P2P_MAX_PEERS)
        self._buffers = {}
        self.signal, self.signal_ptrs = self._alloc("signal", nat.P2P_NUM_CHANNELS * nat.P2P_MAX_PEERS * 4)
        self.cnt, self.cnt_ptrs = self._alloc("counts", self.world * (_MAX_TOT_EXPERT + 1) * 4)
        self.epoch = torch.zeros(8, dtype=torch.int32, device=device)
        self._budget = None
        self._pool = {}
        self.status = nat.status_word(device.index)
        self.ctx = nat.ExchangeContext(self.signal_ptrs, self.epoch, self.me, self.world,
                                       self.status, float(config.wait_timeout_ms()))
        # Nobody may store into a peer's flags before that peer has zeroed them.
        torch.cuda.synchronize(device)
        dist.barrier(group)

    def _alloc(self, name, nbytes):
        nbytes = int(math.ceil(nbytes / 256) * 256)
        t = self._symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        hdl = self._symm_mem.rendezvous(t, group=self.group)
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        self._clear_new(t)
        self._buffers[name] = (t, ptrs, hdl)
        return t, ptrs

    def _clear_new(self, t):
        r"""Zero a fresh symmetric allocation and meet the peers before anybody may store into it.

        Never hand out uninitialised staging memory: kernels that continue after a peer's
        time-out would otherwise act on whatever bits the allocation held.  The barrier matters
        as much as the fill: a peer that is ahead could otherwise deliver rows into the buffer
        before this rank's fill has run, and the fill would wipe them."""
        t.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def buffer(self, name, nbytes):
        r"""Symmetric byte buffer of at least ``nbytes`` (collective when it has to grow; a new
        allocation is cleared and all ranks meet before anybody may store into it)."""
        have = self._buffers.get(name)
        if have is None or have[0].numel() < nbytes:
            torch.cuda.synchronize(self.device)
            self._alloc(name, max(nbytes, 1))
            have = self._buffers[name]
        return have[0], have[1]

    def multicast_ptr(self, name):
        r"""NVSwitch multicast address of a symmetric buffer (0 when the allocation has none)."""
        have = self._buffers.get(name)
        if have is None:
            return 0
        try:
            return int(getattr(have[2], "multicast_ptr", 0) or 0)
        except Exception:  # pylint: disable=broad-except
            return 0

    # ------------------------------------------------------------------ token budget
    def token_budget(self, n_tokens):
        r"""Tokens per rank that every exchange buffer of this group is sized for.

        Fixed by ``FMOE_MAX_TOKENS`` when set; otherwise agreed once, at the first fused call,
        as the maximum of the ranks' batch sizes (one small all-reduce and one host read, never
        again afterwards).  Ranks may bring fewer tokens than the budget — and different
        numbers of them — at any later call.  A rank that brings more cannot be served: the
        peers' buffers are already sized, and growing them is a collective operation the other
        ranks do not know they should join.  That case raises; call :func:`reserve_tokens` on
        all ranks (or set ``FMOE_MAX_TOKENS``) before the larger batch."""
        if self._budget is None:
            fixed = config.max_tokens()
            if fixed > 0:
                self._budget = fixed
            else:
                t = torch.tensor([int(n_tokens)], dtype=torch.int64, device=self.device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
                self._budget = int(t.item())
        if n_tokens > self._budget:
            raise RuntimeError(
                "fastmoe_b200: this rank brings %d tokens to an expert-parallel exchange whose "
                "buffers were sized for %d tokens per rank; call "
                "fastmoe_b200.parallel.symm.reserve_tokens(group, n) on every rank, or set "
                "FMOE_MAX_TOKENS, before using larger batches" % (n_tokens, self._budget))
        return self._budget

    def reserve(self, n_tokens):
        r"""Collective: raise the token budget to the largest ``n_tokens`` any rank asks for."""
        t = torch.tensor([int(n_tokens)], dtype=torch.int64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        self._budget = max(self._budget or 0, int(t.item()))
        return self._budget

    # ------------------------------------------------------------------ per-call leases
    def lease(self, nbytes):
        r"""A symmetric buffer for one layer call (the rows a layer keeps for its backward).

        Buffers come from a pool keyed by size; a new one is a collective allocation, which is
        safe because all ranks run the same sequence of layer calls and hand leases back at the
        same points (end of backward, or end of forward when no graph is recorded)."""
        key = int(math.ceil(max(nbytes, 1) / (1 << 20))) << 20
        free = self._pool.setdefault(key, [])
        if free:
            t, ptrs = free.pop()
        else:
            torch.cuda.synchronize(self.device)
            t = self._symm_mem.empty(key, dtype=torch.uint8, device=self.device)
            hdl = self._symm_mem.rendezvous(t, group=self.group)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
            self._leased_handles = getattr(self, "_leased_handles", [])
            self._leased_handles.append(hdl)
            self._clear_new(t)
        return _Lease(self, key, t, ptrs)

    def item_counters(self, capacity, n_expert):
        r"""Local, self-clearing row counters of the sender warps: one per 128-row block this rank
        can be sending in one exchange (zero between launches)."""
        need = capacity // 128 + 2 * n_expert * self.world + 2
        have = getattr(self, "_item_count", None)
        if have is None or have.numel() < need:
            have = torch.zeros(need, dtype=torch.int32, device=self.device)
            self._item_count = have
        return have

    def gate_flags(self, capacity, n_expert):
        r"""Arrival flags of the receive buffer: int32 ``[blocks][P2P_MAX_PEERS]``."""
        nat = native.get()
        blocks = capacity // 128 + n_expert + 1
        return self.buffer("gate", blocks * nat.P2P_MAX_PEERS * 4)

    def set_timeout_ms(self, ms):
        self.ctx.set_timeout_ms(float(ms))

    def audit(self):
        r"""Host-side audit of the signalling state between steps.  Synchronises the device; call
        it where all ranks of the group are in step (after a barrier), with no layer call in
        flight.  The reference has no counterpart (its exchanges are library collectives); here
        every protocol word has an invariant that must hold again once a step is over:

        * the status word is zero;
        * the grid-completion counters (epoch words 1-5: dispatch, return, reduction, push,
          broadcast) and the sender warps' per-block row counters are back at zero;
        * no flag word — channel flags and the per-block arrival flags of the receive buffer —
          carries an epoch ahead of this rank's own (a peer that ran ahead or a stale buffer);
        * every receive-buffer lease has been handed back.

        Returns a dict with the findings and ``ok``."""
        nat = native.get()
        torch.cuda.synchronize(self.device)
        epoch = [int(v) for v in self.epoch.tolist()]
        exchange_epoch, reduce_epoch = epoch[0], epoch[6]
        signal = self.signal[:nat.P2P_NUM_CHANNELS * nat.P2P_MAX_PEERS * 4].view(torch.int32)
        signal = signal.view(nat.P2P_NUM_CHANNELS, nat.P2P_MAX_PEERS)[:, :self.world]
        ahead = 0
        for chan in range(nat.P2P_NUM_CHANNELS):
            # reduction kernels signal twice per launch: 2 * epoch ("ready") and 2 * epoch + 1 ("done")
            limit = 2 * reduce_epoch + 1 if chan == nat.P2P_CHAN_REDUCE else exchange_epoch
            ahead += int((signal[chan] - limit > 0).sum())
        gate = self._buffers.get("gate")
        if gate is not None:
            flags = gate[0].view(torch.int32).view(-1, nat.P2P_MAX_PEERS)[:, :self.world]
            ahead += int((flags - exchange_epoch > 0).sum())
        counters = getattr(self, "_item_count", None)
        busy_blocks = int((counters != 0).sum()) if counters is not None else 0
        pooled = sum(len(v) for v in self._pool.values())
        leased = len(getattr(self, "_leased_handles", [])) - pooled
        report = {
            "status": int(nat.read_status(self.device.index)),
            "epoch": epoch,
            "completion_counters": epoch[1:6],
            "sender_block_counters_nonzero": busy_blocks,
            "flags_ahead_of_epoch": ahead,
            "leases_outstanding": leased,
        }
        report["ok"] = (report["status"] == 0 and not any(epoch[1:6]) and busy_blocks == 0
                        and ahead == 0 and leased == 0)
        return report


class _Lease:
    r"""One pooled symmetric buffer in use; ``release()`` (or garbage collection) returns it."""

    def __init__(self, ws, key, tensor, ptrs):
        self.ws, self.key, self.tensor, self.ptrs = ws, key, tensor, ptrs

    def release(self):
        if self.tensor is not None:
            self.ws._pool[self.key].append((self.tensor, self.ptrs))  # pylint: disable=protected-access
            self.tensor = None

    def __del__(self):
        try:
            self.release()
        except Exception:  # pylint: disable=broad-except
            pass


def reserve_tokens(group, n_tokens, device=None):
    r"""Collective over ``group``: make the fused expert-parallel path ready for batches of up to
    ``n_tokens`` tokens per rank (the largest value any rank passes wins)."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    ws = get_workspace(group, device)
    if ws is None:
        return None
    return ws.reserve(n_tokens)


def get_workspace(group, device):
    r"""Workspace of ``group`` on ``device`` or ``None`` when symmetric memory cannot be set up."""
    if group is None:
        group = dist.group.WORLD
    key = _group_key(group, device)
    if key in _FAILED:
        return None
    ws = _WORKSPACES.get(key)
    if ws is None:
        try:
            ws = SymmWorkspace(group, device)
        except Exception as exc:  # pylint: disable=broad-except
            _FAILED.add(key)
            if os.environ.get("FMOE_DEBUG", "0") == "1":
                print("[fastmoe_b200] symmetric memory unavailable: %r" % (exc,))
            return None
        _WORKSPACES[key] = ws
    return ws


def _layer_group(layer):
    return layer.moe_group if layer.moe_group is not None else dist.group.WORLD


def fused_available(layer, x):
    r"""True when the peer-to-peer path can serve this layer call."""
    if not config.fused_enabled() or not dist.is_available() or not dist.is_initialized():
        return False
    group = _layer_group(layer)
    if dist.get_backend(group) != "nccl" or dist.get_world_size(group) != layer.world_size:
        return False
    if layer.world_size * layer.num_expert > _MAX_TOT_EXPERT:
        return False
    return get_workspace(group, x.device) is not None


def receive_capacity(n_tokens, k, world):
    r"""Rows reserved for tokens arriving at one rank (see ``config.recv_capacity_factor``);
    ``n_tokens`` is the group's token budget, so every rank computes the same number."""
    factor = config.recv_capacity_factor()
    worst = n_tokens * k * world
    if factor <= 0:
        return worst
    return min(worst, int(math.ceil(factor * n_tokens * k)))


class _Tables:
    r"""Device tables of one exchange, produced by the count-exchange kernel in one tensor."""

    def __init__(self, ws, lec, n_expert, capacity):
        tot = n_expert * ws.world
        w1 = ws.world + 1
        n_blk = capacity // 128 + n_expert
        self.buf = torch.empty(4 * tot + (n_expert + 1) + n_expert * w1 + 2 + n_blk, dtype=torch.int32,
                               device=lec.device)
        ws.ctx.count_exchange(lec, ws.cnt_ptrs, n_expert, capacity, self.buf)
        o = 0
        self.dst_base = self.buf[o:o + tot]; o += tot          # noqa: E702
        self.seg_base = self.buf[o:o + tot]; o += tot          # noqa: E702
        self.blk_base = self.buf[o:o + tot]; o += tot          # noqa: E702
        self.expert_offs = self.buf[o:o + n_expert + 1]; o += n_expert + 1  # noqa: E702
        self.seg_off = self.buf[o:o + n_expert * w1]; o += n_expert * w1    # noqa: E702
        self.total = self.buf[o:o + 1]; o += 1                 # noqa: E702
        self.item_prefix = self.buf[o:o + tot + 1]; o += tot + 1  # noqa: E702
        self.blk_order = self.buf[o:o + n_blk]


def _rows_view(byte_tensor, rows, d, dtype):
    es = torch.empty(0, dtype=dtype).element_size()
    return byte_tensor[:rows * d * es].view(dtype).view(rows, d)


class _DispatchP2P(Function):
    r"""Token rows → the owning ranks' expert segments (forward); row gradients back, summed
    over the k copies of a token (backward)."""

    @staticmethod
    def forward(ctx, x, idx, rank, lec, ws, n_expert, k, capacity, budget):
        nat = native.get()
        d = x.shape[1]
        dev = x.device
        tb = _Tables(ws, lec, n_expert, capacity)
        stage_rows, rows_ptrs = ws.buffer("rows", capacity * d * x.element_size())
        stage_meta, meta_ptrs = ws.buffer("meta", capacity * 8)
        ws.ctx.dispatch_push(x, idx, rank, tb.dst_base, None, rows_ptrs, meta_ptrs, n_expert, k, capacity)
        xs = torch.empty(capacity, d, dtype=x.dtype, device=dev)
        meta = torch.empty(capacity, dtype=torch.int64, device=dev)
        ws.ctx.wait_copy(nat.P2P_CHAN_DISPATCH, stage_rows, stage_meta.view(torch.int64), tb.total, xs, meta)
        ctx.ws = ws
        ctx.k = k
        ctx.n_tok = x.shape[0]
        ctx.budget = budget
        ctx.capacity = capacity
        ctx.save_for_backward(idx, meta, tb.total, rank, tb.dst_base)
        ctx.mark_non_differentiable(tb.expert_offs, meta, tb.total, tb.dst_base)
        return xs, tb.expert_offs, meta, tb.total, tb.dst_base

    @staticmethod
    def backward(ctx, dxs, _g1, _g2, _g3, _g4):
        idx, meta, total, rank, dst_base = ctx.saved_tensors
        ws = ctx.ws
        dxs = dxs.contiguous()
        d = dxs.shape[1]
        stage_ret, ret_ptrs = ws.buffer("ret", ctx.budget * ctx.k * d * dxs.element_size())
        ws.ctx.return_push(dxs, meta, total, ret_ptrs, ctx.budget * ctx.k)
        dx = torch.empty(ctx.n_tok, d, dtype=dxs.dtype, device=dxs.device)
        ws.ctx.wait_combine(stage_ret, idx, None, ctx.k, dx, None, rank=rank, dst_base=dst_base,
                            capacity_rows=ctx.capacity)
        return (dx,) + (None,) * 8


class _CombineP2P(Function):
    r"""Expert output rows → back to their source slots and gate-weighted sum (forward);
    ``d score`` and score-scaled output gradients to the owners (backward)."""

    @staticmethod
    def forward(ctx, ys, score, idx, rank, dst_base, meta, total, ws, n_expert, k, capacity, budget):
        d = ys.shape[1]
        n_tok = idx.numel() // k
        stage_ret, ret_ptrs = ws.buffer("ret", budget * k * d * ys.element_size())
        ws.ctx.return_push(ys, meta, total, ret_ptrs, budget * k)
        out = torch.empty(n_tok, d, dtype=ys.dtype, device=ys.device)
        y_slots = torch.empty(idx.numel(), d, dtype=ys.dtype, device=ys.device)
        ws.ctx.wait_combine(stage_ret, idx, score, k, out, y_slots, rank=rank, dst_base=dst_base,
                            capacity_rows=capacity)
        ctx.ws = ws
        ctx.args = n_expert, k, capacity
        ctx.save_for_backward(y_slots, score, idx, rank, dst_base, total)
        return out

    @staticmethod
    def backward(ctx, dout):
        nat = native.get()
        y_slots, score, idx, rank, dst_base, total = ctx.saved_tensors
        n_expert, k, capacity = ctx.args
        ws = ctx.ws
        dout = dout.contiguous()
        d = dout.shape[1]
        dscore = torch.empty_like(score)
        nat.slot_dot(dout, y_slots, idx, k, dscore)
        ws.ctx.begin_epoch()
        stage_rows, rows_ptrs = ws.buffer("rows", capacity * d * dout.element_size())
        ws.ctx.dispatch_push(dout, idx, rank, dst_base, score, rows_ptrs, [0] * ws.world,
                             n_expert, k, capacity)
        dys = torch.empty(capacity, d, dtype=dout.dtype, device=dout.device)
        ws.ctx.wait_copy(nat.P2P_CHAN_DISPATCH, stage_rows, None, total, dys, None)
        return (dys, dscore) + (None,) * 10


class _FusedEPMLP(Function):
    r"""The whole expert-parallel MLP as one autograd node (activations the GEMM epilogue knows).

    Forward: count exchange → GEMM 1 launch (sender warps dispatch the rows, the GEMM warps
    compute tiles as their rows arrive; + bias, activation) → GEMM 2 whose epilogue stores every
    output row straight into the source rank's return buffer and raises the return flags →
    wait + gate-weighted combine.  Backward: ``d score`` locally; the first input-gradient GEMM
    carries the sender warps for the score-scaled output gradients (and applies the activation
    derivative), then both weight gradients, and the last input-gradient GEMM again pushes its
    rows home, where the k copies of a token are summed.  GEMM 2's result and the expert input
    gradient never exist as local tensors; received rows are never copied out of the buffer
    they landed in.
    """

    @staticmethod
    def forward(ctx, x, score, w1, b1, w2, b2, idx, rank, lec, my_offs, pos, ws, n_expert, k,
                capacity, budget, act):
        from ..ops import grouped_gemm as gg
        d = x.shape[1]
        h = w1.shape[1]
        dev = x.device
        es = x.element_size()
        code = gg.ACT_CODES[act]
        with fused_range("ep.counts"):
            tb = _Tables(ws, lec, n_expert, capacity)
        lease = ws.lease(capacity * d * es + capacity * 8)
        xs = _rows_view(lease.tensor, capacity, d, x.dtype)
        meta = lease.tensor[capacity * d * es:capacity * d * es + capacity * 8].view(torch.int64)
        meta_ptrs = [p + capacity * d * es for p in lease.ptrs]
        _flags, flag_ptrs = ws.gate_flags(capacity, n_expert)
        send = dict(x=x, pos=pos, my_offs=my_offs, dst_base=tb.dst_base, seg_base=tb.seg_base,
                    blk_base=tb.blk_base, rows_ptrs=lease.ptrs, meta_ptrs=meta_ptrs,
                    flag_ptrs=flag_ptrs, n_expert=n_expert, k=k, capacity=capacity,
                    item_prefix=tb.item_prefix, item_count=ws.item_counters(capacity, n_expert))
        with fused_range("ep.dispatch_gemm1"):
            a = torch.empty(capacity, h, dtype=x.dtype, device=dev)
            pre = gg.pre_buffer(capacity, h, n_expert, x.dtype, dev) if code != 0 else a
            ws.ctx.gemm_ep(gg.MODE_NT, xs, w1, tb.expert_offs, out=a, bias=b1,
                           pre_out=pre if code != 0 else None, act=code, send=send,
                           gate_flag_ptrs=flag_ptrs, seg_off=tb.seg_off, blk_order=tb.blk_order,
                           trace=new_ep_trace(dev) if config.ep_trace() else None)
        with fused_range("ep.gemm2_push_combine"):
            n_slots_cap = budget * k
            stage_ret, ret_ptrs = ws.buffer("ret", n_slots_cap * d * es)
            ws.ctx.gemm_ep(gg.MODE_NT, a, w2, tb.expert_offs, bias=b2, push_meta=meta,
                           ret_ptrs=ret_ptrs, push_slots=n_slots_cap)
            n_tok = x.shape[0]
            out = torch.empty(n_tok, d, dtype=x.dtype, device=dev)
            y_slots = torch.empty(idx.numel(), d, dtype=x.dtype, device=dev)
            ws.ctx.wait_combine(stage_ret, idx, score, k, out, y_slots, rank=rank,
                                dst_base=tb.dst_base, capacity_rows=capacity)

        ctx.ws = ws
        ctx.args = n_expert, k, capacity, budget, act, n_tok
        ctx.lease = lease
        ctx.save_for_backward(xs, pre, a, w1, w2, tb.buf, meta, idx, my_offs, pos, score, y_slots, rank)
        ctx.tables = tb
        if not any(ctx.needs_input_grad):
            lease.release()  # nothing will run backward through this call
        return out

    @staticmethod
    def backward(ctx, dout):
        from ..ops import grouped_gemm as gg
        nat = native.get()
        (xs, pre, a, w1, w2, _tbuf, meta, idx, my_offs, pos, score, y_slots, rank) = ctx.saved_tensors
        n_expert, k, capacity, budget, act, n_tok = ctx.args
        tb = ctx.tables
        ws = ctx.ws
        dout = dout.contiguous()
        d = dout.shape[1]
        h = w1.shape[1]
        es = dout.element_size()
        code = gg.ACT_CODES[act]
        dscore = torch.empty_like(score)
        nat.slot_dot(dout, y_slots, idx, k, dscore)
        ws.ctx.begin_epoch()
        # The gradient rows land in a buffer all layers share and are read in place by the next
        # two GEMMs: no peer writes it again before it has combined what this rank pushes at the
        # very end of this backward (or, when no input gradient is wanted, before the count
        # exchange of the next forward).
        stage_rows, rows_ptrs = ws.buffer("rows_bwd", capacity * d * es)
        dys = _rows_view(stage_rows, capacity, d, dout.dtype)
        _flags, flag_ptrs = ws.gate_flags(capacity, n_expert)
        send = dict(x=dout, pos=pos, my_offs=my_offs, dst_base=tb.dst_base, seg_base=tb.seg_base,
                    blk_base=tb.blk_base, scale=score, rows_ptrs=rows_ptrs, meta_ptrs=None,
                    flag_ptrs=flag_ptrs, n_expert=n_expert, k=k, capacity=capacity,
                    item_prefix=tb.item_prefix, item_count=ws.item_counters(capacity, n_expert))
        da = torch.empty(capacity, h, dtype=dout.dtype, device=dout.device)
        ws.ctx.gemm_ep(gg.MODE_NN, dys, w2, tb.expert_offs, out=da, aux=pre if code != 0 else None,
                       act=code, epi=gg.EPI_DACT if code != 0 else gg.EPI_BIAS_ACT, send=send,
                       gate_flag_ptrs=flag_ptrs, seg_off=tb.seg_off, blk_order=tb.blk_order)
        dw2, db2 = gg.wgrad(dys, a, tb.expert_offs, n_expert, with_bias_grad=True)
        dw1, db1 = gg.wgrad(da, xs, tb.expert_offs, n_expert, with_bias_grad=True)
        dx = None
        if ctx.needs_input_grad[0]:
            n_slots_cap = budget * k
            stage_ret, ret_ptrs = ws.buffer("ret", n_slots_cap * d * es)
            ws.ctx.gemm_ep(gg.MODE_NN, da, w1, tb.expert_offs, push_meta=meta, ret_ptrs=ret_ptrs,
                           push_slots=n_slots_cap)
            dx = torch.empty(n_tok, d, dtype=dout.dtype, device=dout.device)
            ws.ctx.wait_combine(stage_ret, idx, None, k, dx, None, rank=rank, dst_base=tb.dst_base,
                                capacity_rows=capacity)
        ctx.lease.release()
        return (dx, dscore, dw1, db1, dw2, db2) + (None,) * 11


def moe_mlp_forward(layer, x, gate_idx, gate_score):
    r"""Fused ``FMoETransformerMLP`` call under expert parallelism (``world_size > 1``)."""
    from ..ops import fused
    from ..transformer import activation_kind
    nat = native.get()
    ws = get_workspace(_layer_group(layer), x.device)
    k = gate_idx.shape[1]
    n_expert = layer.num_expert
    budget = ws.token_budget(x.shape[0])
    idx = gate_idx.contiguous().view(-1)
    score = gate_score.reshape(-1).to(x.dtype)
    lec, rank, my_offs, pos = nat.route_pos(idx, n_expert * ws.world)
    if config.debug_bounds():
        from ..utils.profiling import check_routing
        check_routing(idx, rank, lec, n_expert * ws.world)
    capacity = receive_capacity(budget, k, ws.world)
    act = activation_kind(layer.experts.activation)
    if act is not None:
        e = layer.experts
        return _FusedEPMLP.apply(x.contiguous(), score, e.htoh4.weight, e.htoh4.bias, e.h4toh.weight,
                                 e.h4toh.bias, idx, rank, lec, my_offs, pos, ws, n_expert, k,
                                 capacity, budget, act)
    xs, expert_offs, meta, total, dst_base = _DispatchP2P.apply(
        x.contiguous(), idx, rank, lec, ws, n_expert, k, capacity, budget)
    ys = fused.expert_mlp(layer, xs, expert_offs)
    return _CombineP2P.apply(ys, score, idx, rank, dst_base, meta, total, ws, n_expert, k, capacity,
                             budget)


# ------------------------------------------------------------------------------------------
# Gradient all-reduce of replicated parameters
# ------------------------------------------------------------------------------------------
_AR_DTYPES = (torch.bfloat16, torch.float16, torch.float32)
_AR_MAX_BYTES = 1024 * 1024 * 1024
# Above this size the two-shot kernel (each rank reduces one slice and writes it to all peers)
# moves fewer bytes over NVLink than the one-shot kernel (each rank reads every peer in full).
_AR_TWO_SHOT_BYTES = 512 * 1024


def _ar_buffer_bytes(nbytes):
    return (nbytes + 15) // 16 * 16


def _two_shot(nbytes, world):
    return world > 2 and nbytes >= _AR_TWO_SHOT_BYTES or nbytes >= 8 * _AR_TWO_SHOT_BYTES


def _run_allreduce(ws, ptrs, out, n, nbytes, scale):
    r"""The reduction kernel for a filled "allreduce" buffer: through NVSwitch (``multimem``
    in-switch reduction) when ``FMOE_USE_NVLS=1`` and the buffer has a multicast mapping, else
    with plain peer loads / stores (one-shot for small buckets, two-shot from 512 KiB)."""
    if config.use_nvls() and ws.world > 1:
        mc = ws.multicast_ptr("allreduce")
        if mc != 0:
            ws.ctx.allreduce_multimem(mc, ptrs[ws.me], out, float(scale))
            return
    ws.ctx.allreduce(ptrs, out, n, float(scale), _two_shot(nbytes, ws.world))


def allreduce_grads(grads, comm, scale, fp32_accumulate=False):  # pylint: disable=unused-argument
    r"""Sum ``grads`` over ``comm`` in place with the peer-to-peer kernels (one-shot for small
    buckets, two-shot from 512 KiB).

    Sums are formed in rank order with fp32 accumulation, so the result is bit-identical on
    all ranks and ``fp32_accumulate`` is implied.  Returns ``False`` (caller
    falls back to the collective library) for unsupported dtypes, very large buckets or when
    no symmetric workspace exists for the group.
    """
    if not config.fused_enabled() or not grads:
        return False
    dtype = grads[0].dtype
    if dtype not in _AR_DTYPES or dist.get_backend(comm) != "nccl":
        return False
    n = sum(g.numel() for g in grads)
    if n * grads[0].element_size() > _AR_MAX_BYTES:
        return False
    ws = get_workspace(comm, grads[0].device)
    if ws is None:
        return False
    nbytes = n * grads[0].element_size()
    with fused_range("allreduce"):
        return _allreduce_grads(ws, grads, n, nbytes, dtype, scale)


def _allreduce_grads(ws, grads, n, nbytes, dtype, scale):
    buf, ptrs = ws.buffer("allreduce", _ar_buffer_bytes(nbytes))
    flat = buf[:nbytes].view(dtype)
    views = []
    offset = 0
    for g in grads:
        views.append(flat[offset:offset + g.numel()].view_as(g))
        offset += g.numel()
    torch._foreach_copy_(views, grads)  # pylint: disable=protected-access
    out = torch.empty(n, dtype=dtype, device=grads[0].device)
    _run_allreduce(ws, ptrs, out, n, nbytes, scale)
    outs = []
    offset = 0
    for g in grads:
        outs.append(out[offset:offset + g.numel()].view_as(g))
        offset += g.numel()
    torch._foreach_copy_(grads, outs)  # pylint: disable=protected-access
    return True


def allreduce_flat(flat, comm, scale=1.0):
    r"""Sum of a 1-D tensor over ``comm`` with the peer-to-peer all-reduce kernels, or ``None`` when
    that path is not available (caller falls back to the collective library).

    Used for the shadow-expert traffic: a parameter *broadcast* is the sum of the owner's values
    and zeros everywhere else, the gradient *reduce* is a sum of which only the owner keeps the
    result.
    """
    if not flat.is_cuda or not config.fused_enabled() or flat.dtype not in _AR_DTYPES:
        return None
    if comm is None:
        comm = dist.group.WORLD
    if dist.get_backend(comm) != "nccl" or flat.numel() * flat.element_size() > _AR_MAX_BYTES:
        return None
    ws = get_workspace(comm, flat.device)
    if ws is None:
        return None
    n = flat.numel()
    nbytes = n * flat.element_size()
    buf, ptrs = ws.buffer("allreduce", _ar_buffer_bytes(nbytes))
    buf[:nbytes].view(flat.dtype).copy_(flat.reshape(-1))
    out = torch.empty(n, dtype=flat.dtype, device=flat.device)
    _run_allreduce(ws, ptrs, out, n, nbytes, scale)
    return out


def broadcast_flat(flat, owner, comm):
    r"""The owner's 1-D tensor on every rank of ``comm`` (``owner`` is a rank inside the group),
    pushed by the owner with one peer-to-peer write per peer; ``None`` when that path is not
    available.  ``flat`` must have the same length and dtype everywhere; its values only matter
    on the owner.  Parity: the ``ncclBcast`` of shadow-expert parameters,
    ``cuda/fastermoe/smart_schedule.h:182``."""
    if not flat.is_cuda or not config.fused_enabled():
        return None
    if comm is None:
        comm = dist.group.WORLD
    nbytes = flat.numel() * flat.element_size()
    if dist.get_backend(comm) != "nccl" or nbytes == 0 or nbytes > _AR_MAX_BYTES:
        return None
    ws = get_workspace(comm, flat.device)
    if ws is None:
        return None
    padded = _ar_buffer_bytes(nbytes)
    _buf, ptrs = ws.buffer("broadcast", padded)
    src = flat.detach().reshape(-1).contiguous()
    if padded != nbytes or src.data_ptr() % 16 != 0:
        grown = torch.zeros(padded // flat.element_size(), dtype=flat.dtype, device=flat.device)
        grown[:flat.numel()] = src
        src = grown
    out = torch.empty_like(src)
    ws.ctx.broadcast(src, ptrs, out, int(owner))
    return out[:flat.numel()]


def reduce_flat_to_owner(flat, owner, comm):
    r"""Sum of the ranks' 1-D tensors, formed on ``owner`` only (peer-to-peer loads by the owner);
    returns the sum there and zeros elsewhere, or ``None`` when the path is not available.
    Parity: ``reduce_grad`` (``cuda/fastermoe/smart_schedule.cpp:41-63``)."""
    if not flat.is_cuda or not config.fused_enabled() or flat.dtype not in _AR_DTYPES:
        return None
    if comm is None:
        comm = dist.group.WORLD
    nbytes = flat.numel() * flat.element_size()
    if dist.get_backend(comm) != "nccl" or nbytes == 0 or nbytes > _AR_MAX_BYTES:
        return None
    ws = get_workspace(comm, flat.device)
    if ws is None:
        return None
    n = flat.numel()
    buf, ptrs = ws.buffer("allreduce", _ar_buffer_bytes(nbytes))
    buf[:nbytes].view(flat.dtype).copy_(flat.reshape(-1))
    out = torch.zeros(n, dtype=flat.dtype, device=flat.device)
    ws.ctx.reduce_to_root(ptrs, out, n, int(owner))
    return out


def allgather_rows(inp, comm, out=None):
    r"""``out = cat([inp of rank 0, inp of rank 1, ...])`` with peer-to-peer stores, or ``None``
    when that path is not available (caller uses the collective library).

    Parity: the all-gather of ``fmoe/functions.py:308-329`` (``AllGather.forward``,
    ``Slice.backward``), which the reference follows with a device synchronisation.
    """
    if not inp.is_cuda or not config.fused_enabled():
        return None
    if comm is None:
        comm = dist.group.WORLD
    nbytes = inp.numel() * inp.element_size()
    if (dist.get_backend(comm) != "nccl" or nbytes == 0 or nbytes % 16 != 0
            or nbytes * dist.get_world_size(comm) > _AR_MAX_BYTES):
        return None
    ws = get_workspace(comm, inp.device)
    if ws is None:
        return None
    inp = inp.contiguous()
    if inp.data_ptr() % 16 != 0:
        inp = inp.clone()
    _buf, ptrs = ws.buffer("allgather", nbytes * ws.world)
    if out is None:
        out = inp.new_empty((ws.world * inp.shape[0],) + tuple(inp.shape[1:]))
    ws.ctx.allgather(inp, ptrs, out)
    return out


def swipe_round(idx, capacity, n_expert, n_worker, bias, comm=None):
    r"""One SWIPE round entirely on the device: ``(balanced ids, capacity left)`` — both CUDA
    tensors — or ``None`` when the peer-to-peer path is not available.

    ``idx``: int64 global expert ids of one choice column; ``capacity``: int64 ``[1]`` tokens this
    worker can still accept.  Parity: ``cuda/balancing.cu:83-186``; no count is read on the host,
    so a gate built on it can be captured in a CUDA graph."""
    if not idx.is_cuda or not config.fused_enabled():
        return None
    if comm is None:
        comm = dist.group.WORLD
    if dist.get_backend(comm) != "nccl" or dist.get_world_size(comm) != n_worker:
        return None
    ws = get_workspace(comm, idx.device)
    if ws is None:
        return None
    nat = native.get()
    idx = idx.reshape(-1).contiguous()
    worker = torch.div(idx, n_expert, rounding_mode="floor")
    want, _rank = nat.route(worker, n_worker)
    cap = capacity.reshape(1).to(device=idx.device, dtype=torch.int64)
    _buf, ptrs = ws.buffer("swipe", 2 * ws.world * (ws.world + 1) * 8)
    quota, left = ws.ctx.swipe_exchange(want, cap, ptrs)
    return nat.swipe_reassign(idx, quota, n_expert, int(bias)), left


def capacity_grant(lec, cap, n_expert, comm=None):
    r"""``(new_lec, new_gec)`` (int64) of a global capacity limit with ONE peer-to-peer exchange,
    or ``None`` when that path is not available.

    ``lec``: int32 ``[world * n_expert]`` slots this rank wants to send to every global expert;
    ``cap``: int32 ``[n_expert]`` capacities of this rank's experts.  Parity: the count
    all-to-all → ``limit_by_capacity`` → grant all-to-all sequence of
    ``fmoe/gates/utils.py:9-26``; grants are handed out in rank order, as there.
    """
    if not lec.is_cuda or not config.fused_enabled():
        return None
    if comm is None:
        comm = dist.group.WORLD
    if dist.get_backend(comm) != "nccl":
        return None
    ws = get_workspace(comm, lec.device)
    if ws is None:
        return None
    width = (ws.world + 1) * n_expert
    if ws.world * width * 4 > 200 * 1024:
        return None
    _buf, ptrs = ws.buffer("capacity", 2 * ws.world * width * 4)
    new_lec, new_gec = ws.ctx.capacity_grant(lec.contiguous(), cap.contiguous(), ptrs, n_expert)
    return new_lec, new_gec
