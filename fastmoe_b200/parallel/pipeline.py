r"""
Pipeline parallelism around MoE stages: a 1F1B runner that carries the gates' balance loss.

The reference has no pipeline engine of its own; it patches Megatron-LM's so that every stage
back-propagates the balance loss of its own MoE layers together with the gradient it receives
from the next stage, scaled by ``1 / pipeline_size`` (``examples/megatron/v3.0.2.patch:232-397``,
``fmoe/megatron/patch.py:45,121``), and it makes the *gate group* the set of ranks of one stage
(``fmoe/megatron/distributed.py:26-37``).  This module provides the same schedule and the same
loss threading without Megatron, so that hybrid pipeline × expert parallelism can be run and
tested with this package alone.  Activations and gradients travel with ``torch.distributed``
point-to-point operations (the collective library; the MoE exchange inside a stage is
independent of it), and the paired "send one way, receive the other way" steps are posted
together so that neighbouring stages cannot block each other.

Layout of the ranks: ``world = n_stages × stage_size``; rank ``r`` runs stage ``r // stage_size``
and talks to ``r ± stage_size``; the ``stage_size`` ranks of a stage form its expert-parallel /
gate / data-parallel group (:func:`build_stage_groups`).
"""
import torch
import torch.distributed as dist


def build_stage_groups(n_stages):
    r"""``(stage, stage_group, prev_rank, next_rank)`` for the calling rank.

    Every rank must call this (group creation is collective).  ``prev_rank`` / ``next_rank``
    are ``None`` at the ends of the pipeline.
    """
    world, rank = dist.get_world_size(), dist.get_rank()
    assert world % n_stages == 0, "world size must be a multiple of the number of stages"
    stage_size = world // n_stages
    mine = None
    for s in range(n_stages):
        group = dist.new_group(list(range(s * stage_size, (s + 1) * stage_size)))
        if rank // stage_size == s:
            mine = group
    stage = rank // stage_size
    prev_rank = rank - stage_size if stage > 0 else None
    next_rank = rank + stage_size if stage < n_stages - 1 else None
    return stage, mine, prev_rank, next_rank


def collect_balance_loss(module):
    r"""Mean of the balance losses the gates of ``module`` recorded in the last forward
    (``None`` when no gate has one).  Reading clears them, as Megatron's patched step does."""
    losses = []
    for m in module.modules():
        gate = getattr(m, "gate", None)
        if gate is not None and getattr(gate, "has_loss", False):
            losses.append(gate.get_loss(clear=True).reshape(1).float())
    if not losses:
        return None
    return torch.cat(losses).mean()


class PipelineRunner:
    r"""Non-interleaved 1F1B over ``n_micro`` micro-batches for one stage.

    ``stage_module(x)`` maps the stage's input activation to its output activation; on the
    first stage ``x`` is the micro-batch itself, on the last stage ``loss_fn(output, target)``
    turns the output into a scalar.  ``balance_weight`` > 0 adds, on every stage,
    ``balance_weight / n_stages`` times the mean balance loss of the stage's gates to what is
    back-propagated.  Gradients accumulate in ``.grad`` over the micro-batches, each scaled by
    ``1 / n_micro``; reduce them afterwards with ``DistributedGroupedDataParallel`` built on the
    stage group.
    """

    def __init__(self, stage_module, stage, n_stages, prev_rank, next_rank, act_shape, act_dtype,
                 loss_fn=None, balance_weight=0.0, device=None):
        self.module = stage_module
        self.stage, self.n_stages = stage, n_stages
        self.prev_rank, self.next_rank = prev_rank, next_rank
        self.act_shape, self.act_dtype = tuple(act_shape), act_dtype
        self.loss_fn = loss_fn
        self.balance_weight = float(balance_weight)
        self.device = device if device is not None else torch.device("cpu")
        self.first, self.last = stage == 0, stage == n_stages - 1
        assert not self.last or loss_fn is not None, "the last stage needs a loss function"

    # ------------------------------------------------------------------ point-to-point steps
    def _new(self):
        return torch.empty(self.act_shape, dtype=self.act_dtype, device=self.device)

    def _exchange(self, send_to_next=None, send_to_prev=None, recv_from_prev=False, recv_from_next=False):
        ops, got_prev, got_next = [], None, None
        if send_to_prev is not None and not self.first:
            ops.append(dist.P2POp(dist.isend, send_to_prev.contiguous(), self.prev_rank))
        if recv_from_prev and not self.first:
            got_prev = self._new()
            ops.append(dist.P2POp(dist.irecv, got_prev, self.prev_rank))
        if send_to_next is not None and not self.last:
            ops.append(dist.P2POp(dist.isend, send_to_next.contiguous(), self.next_rank))
        if recv_from_next and not self.last:
            got_next = self._new()
            ops.append(dist.P2POp(dist.irecv, got_next, self.next_rank))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        return got_prev, got_next

    # ------------------------------------------------------------------ compute steps
    def _forward(self, received, micro, target):
        if self.first:
            x = micro
        else:
            x = received.requires_grad_(True)
        out = self.module(x)
        bal = collect_balance_loss(self.module) if self.balance_weight > 0 else None
        if self.last:
            out = self.loss_fn(out, target)
        return x, out, bal

    def _backward(self, x, out, bal, out_grad, n_micro):
        extra = None
        if bal is not None:
            extra = bal * (self.balance_weight / self.n_stages / n_micro)
        if self.last:
            total = out / n_micro
            if extra is not None:
                total = total + extra.to(total.dtype)
            total.backward()
        elif extra is not None:
            # the received gradient already carries the 1 / n_micro of the last stage's loss
            torch.autograd.backward([out, extra.to(out.dtype)], [out_grad, None])
        else:
            out.backward(out_grad)
        if self.first or x.grad is None:
            return None
        return x.grad

    # ------------------------------------------------------------------ the schedule
    def run(self, micro_batches=None, targets=None, n_micro=None):
        r"""One optimisation step's worth of forward and backward passes.

        ``micro_batches``: list of inputs (first stage only); ``targets``: list of targets (last
        stage only); ``n_micro`` must be given on the middle stages.  Returns the mean loss on
        the last stage and ``None`` elsewhere.
        """
        if n_micro is None:
            n_micro = len(micro_batches if micro_batches is not None else targets)
        warmup = min(self.n_stages - self.stage - 1, n_micro)
        steady = n_micro - warmup
        stash, losses = [], []
        fwd_i = 0

        def fwd(received):
            nonlocal fwd_i
            micro = micro_batches[fwd_i] if self.first else None
            target = targets[fwd_i] if self.last else None
            fwd_i += 1
            item = self._forward(received, micro, target)
            if self.last:
                losses.append(item[1].detach())
            return item

        for _ in range(warmup):
            received, _ = self._exchange(recv_from_prev=True)
            item = fwd(received)
            self._exchange(send_to_next=item[1].detach())
            stash.append(item)
        received = None
        if steady > 0:
            received, _ = self._exchange(recv_from_prev=True)
        for i in range(steady):
            item = fwd(received)
            stash.append(item)
            # send the activation forward and receive the gradient of the oldest micro-batch
            _, out_grad = self._exchange(send_to_next=None if self.last else item[1].detach(),
                                         recv_from_next=True)
            x, out, bal = stash.pop(0)
            in_grad = self._backward(x, out, bal, out_grad, n_micro)
            if i == steady - 1:
                self._exchange(send_to_prev=in_grad)
            else:
                received, _ = self._exchange(send_to_prev=in_grad, recv_from_prev=True)
        for _ in range(warmup):
            _, out_grad = self._exchange(recv_from_next=True)
            x, out, bal = stash.pop(0)
            in_grad = self._backward(x, out, bal, out_grad, n_micro)
            self._exchange(send_to_prev=in_grad)
        if self.last:
            return torch.stack(losses).mean()
        return None
