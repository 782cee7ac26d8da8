r"""
Data parallelism with a different all-reduce group per parameter.

Parity: ``fmoe/distributed.py:10-114``.  A parameter's attribute ``dp_comm`` names the
group that averages its gradient: ``'dp'`` (default), ``'gate'``, ``'world'``, ``'moe'`` or
any ``<name>`` passed as ``<name>_group=`` to the constructor; parameters tagged with a name
that has no group (``'none'`` — the experts under expert parallelism) are left alone.

Differences from the reference: gradients of one ``(dp_comm, dtype)`` bucket live in one
flat buffer that is reduced in place — on B200s by the peer-to-peer/NVSwitch kernel of
:mod:`fastmoe_b200.ops.allreduce`, which also applies the ``1/size`` scale and the optional
fp32 accumulation in the same pass — instead of flatten → all-reduce → unflatten → copy
(``fmoe/distributed.py:63-75``).
"""
import torch
import torch.distributed as dist
import torch.nn as nn

from .parallel.comm import get_rank_0_in_comm, get_torch_default_comm


def _bucket_params(params, need_grad):
    buckets = {}
    for p in params:
        if need_grad and (not p.requires_grad or p.grad is None):
            continue
        key = (getattr(p, "dp_comm", "dp"), p.dtype)
        buckets.setdefault(key, []).append(p)
    return buckets


class _ReduceHandle:
    r"""Returned by ``allreduce_gradients(async_op=True)``."""

    def __init__(self, stream):
        self._stream = stream

    def wait(self):
        if self._stream is not None:
            torch.cuda.current_stream().wait_stream(self._stream)
            self._stream = None


class DistributedGroupedDataParallel(nn.Module):
    r"""Wraps ``module``; call :meth:`allreduce_params` after backward.

    ``auto_allreduce`` is not implemented in the reference either.  ``need_sync`` broadcasts
    every bucket from the first member of its group at construction.
    """

    def __init__(self, module, auto_allreduce=False, need_sync=True, status_check_interval=100,
                 **kwargs):
        assert not auto_allreduce, "Automatic all-reduce is not implemented yet"
        super().__init__()
        self.module = module
        self.comms = {}
        self._side_stream = None
        # Every `status_check_interval` reductions the device status word is read (one
        # synchronisation): a peer time-out or a receive-buffer overflow reported by any kernel
        # since the last check raises here instead of training on.  0 switches the check off.
        self.status_check_interval = status_check_interval
        self._reductions = 0
        for name, group in kwargs.items():
            if name.endswith("_group"):
                self.comms[name[:-len("_group")]] = group
        for name in ("dp", "gate", "moe", "world"):
            if name not in self.comms:
                self.comms[name] = get_torch_default_comm()
        if need_sync:
            self._sync_params()

    # -------------------------------------------------------------- gradient reduction
    def allreduce_gradients(self, no_scale=False, reduce_after=False, fp32_allreduce=False,
                            async_op=False):
        r"""Average (or sum, with ``no_scale``) gradients inside each parameter's group.

        ``async_op=True`` (CUDA only; not in the reference) issues the reductions on a side
        stream behind everything already queued on the current stream and returns a handle;
        ``handle.wait()`` makes the current stream wait for them.  Work that does not touch
        the reduced gradients — typically the optimizer step of the expert parameters, which
        are not reduced under expert parallelism — can be queued in between and overlaps the
        latency-bound all-reduce.  ``wait()`` must come before the next forward of the model.
        The fork and the join are stream dependencies, so they can be captured in a CUDA graph.
        """
        if async_op and torch.cuda.is_available():
            main = torch.cuda.current_stream()
            if self._side_stream is None:
                self._side_stream = torch.cuda.Stream()
            side = self._side_stream
            side.wait_stream(main)
            with torch.cuda.stream(side):
                self.allreduce_gradients(no_scale, reduce_after, fp32_allreduce)
            return _ReduceHandle(side)
        if async_op:
            # no GPU: reduce now and hand back a handle whose wait() has nothing left to do
            self.allreduce_gradients(no_scale, reduce_after, fp32_allreduce)
            return _ReduceHandle(None)
        from .ops import allreduce as _ar
        self._reductions += 1
        if (self.status_check_interval and self._reductions % self.status_check_interval == 0
                and torch.cuda.is_available() and not torch.cuda.is_current_stream_capturing()):
            from .utils import check_device_status
            check_device_status()
        for (dp_comm, dtype), group_params in _bucket_params(self.module.parameters(), True).items():
            if dp_comm not in self.comms:
                continue
            comm = self.comms[dp_comm]
            size = dist.get_world_size(comm)
            scale = 1.0 if no_scale else 1.0 / size
            grads = [p.grad.data for p in group_params]
            if _ar.try_fused_allreduce(grads, comm, scale, fp32_accumulate=fp32_allreduce):
                continue
            flat = torch.cat([g.reshape(-1) for g in grads])
            if fp32_allreduce and dtype != torch.float32:
                flat = flat.float()
            if not no_scale and not reduce_after:
                flat /= size
            dist.all_reduce(flat, group=comm)
            if not no_scale and reduce_after:
                flat /= size
            offset = 0
            for g in grads:
                g.copy_(flat[offset:offset + g.numel()].view_as(g))
                offset += g.numel()

    def allreduce_params(self, *args, **kwargs):
        r"""Alias kept because Megatron versions call one name or the other."""
        return self.allreduce_gradients(*args, **kwargs)

    # -------------------------------------------------------------- initial sync
    def _sync_params(self):
        for (dp_comm, _dtype), group_params in _bucket_params(self.module.parameters(), False).items():
            if dp_comm not in self.comms:
                continue
            comm = self.comms[dp_comm]
            datas = [p.data for p in group_params]
            flat = torch.cat([d.reshape(-1) for d in datas])
            dist.broadcast(flat, get_rank_0_in_comm(comm), group=comm)
            offset = 0
            for d in datas:
                d.copy_(flat[offset:offset + d.numel()].view_as(d))
                offset += d.numel()

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)
