r"""
Tracing and timing helpers.

The reference has none (its ``cuda/utils/timer.hh`` is commented out and
``tests/benchmark_mlp.py:92-106`` times with ``time.time()`` without synchronising).  Here:
NVTX ranges for every fused path, CUDA-event timers whose result is reduced with MAX over the
ranks of a group (the way every multi-GPU number of this project is reported), and a JSON-lines
logger for benchmark output.
"""
import contextlib
import json
import time

import torch
import torch.distributed as dist


@contextlib.contextmanager
def nvtx_range(name):
    r"""NVTX range on the current thread (no-op without CUDA)."""
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


@contextlib.contextmanager
def fused_range(name):
    r"""NVTX range used inside the framework's fused paths; active only with ``FMOE_NVTX=1``
    so that the default path pays one environment lookup."""
    from .. import config
    if config.nvtx_enabled():
        with nvtx_range("fmoe:" + name):
            yield
    else:
        yield


_ep_traces = []
EP_TRACE_SLOTS = 10
_EP_TRACE_KEEP = 64


def new_ep_trace(device):
    r"""A zeroed trace buffer (ten int64 per SM) for one launch of the fused dispatch + GEMM
    kernel; the last ``64`` buffers are kept for :func:`ep_trace_summary`."""
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    buf = torch.zeros(sms * EP_TRACE_SLOTS, dtype=torch.int64, device=device)
    _ep_traces.append(buf)
    del _ep_traces[:-_EP_TRACE_KEEP]
    return buf


def summarize_ep_trace(stamps):
    r"""Phase durations in microseconds from one trace buffer (``[ctas, 10]``: nanosecond stamps
    entry, first rows available, sender done, exit, then for the first unit of the CTA's first
    sender warp: slot ids loaded, stores issued, fence passed, rows counted; 0 = the CTA never
    reached that phase; then the nanoseconds the TMA producer waited for rows over all its tiles
    and the number of tiles that waited more than a microsecond).

    ``launch_skew``: latest entry − earliest entry; ``first_rows``: how long CTAs waited for the
    rows of their first tile (median, max); ``sender``: entry → last sender warp done (max);
    ``kernel``: earliest entry → latest exit; ``first_unit``: medians over CTAs, from CTA entry;
    ``rows_wait``: producer wait per CTA summed over its tiles (median, max) and tiles that waited.
    """
    t = stamps.reshape(-1, EP_TRACE_SLOTS).cpu().double()
    ran = t[:, 0] > 0
    if not bool(ran.any()):
        return None
    t = t[ran]
    start = float(t[:, 0].min())
    out = {"ctas": int(t.shape[0]),
           "launch_skew_us": (float(t[:, 0].max()) - start) / 1e3,
           "kernel_us": (float(t[:, :4].max()) - start) / 1e3}
    gated = t[:, 1] > 0
    if bool(gated.any()):
        wait = (t[gated, 1] - t[gated, 0]) / 1e3
        out["first_rows_us"] = {"median": float(wait.median()), "max": float(wait.max())}
        out["rows_wait_us"] = {"median": float(t[gated, 8].median()) / 1e3, "max": float(t[gated, 8].max()) / 1e3,
                               "tiles_waited": int(t[gated, 9].sum())}
    sent = t[:, 2] > 0
    if bool(sent.any()):
        out["sender_us"] = (float(t[sent, 2].max()) - start) / 1e3
    unit = t[:, 7] > 0
    if bool(unit.any()):
        rel = (t[unit, 4:8] - t[unit, 0:1]) / 1e3
        med = rel.median(dim=0).values
        out["first_unit_us"] = {"ids_loaded": float(med[0]), "stores_issued": float(med[1]),
                                "fenced": float(med[2]), "counted": float(med[3])}
    return out


def ep_trace_summary(clear=True):
    r"""Summaries of the launches traced under ``FMOE_EP_TRACE=1`` (oldest first).  Synchronises."""
    torch.cuda.synchronize()
    out = [s for s in (summarize_ep_trace(b) for b in _ep_traces) if s is not None]
    if clear:
        _ep_traces.clear()
    return out


def check_routing(idx, rank, counts, tot_expert, offs=None, capacity=None):
    r"""Host-side validation of a routing table (``FMOE_DEBUG_BOUNDS=1``); raises ``ValueError``.

    ``idx``: expert id per slot (``-1`` = dropped); ``rank``: rank of the slot inside its
    expert; ``counts[e]``: slots kept for expert ``e``; ``offs``: exclusive prefix of the
    counts (optional); ``capacity``: rows of the buffer the offsets index (optional).
    """
    idx = idx.reshape(-1).long().cpu()
    rank = rank.reshape(-1).long().cpu()
    counts = counts.reshape(-1).long().cpu()
    if idx.numel() and (int(idx.min()) < -1 or int(idx.max()) >= tot_expert):
        raise ValueError("expert id out of range [-1, %d): min %d max %d" %
                         (tot_expert, int(idx.min()), int(idx.max())))
    kept = idx >= 0
    want = torch.bincount(idx[kept], minlength=tot_expert)[:tot_expert]
    if not torch.equal(want, counts[:tot_expert]):
        raise ValueError("expert counts do not match the expert ids")
    if kept.any():
        if int(rank[kept].min()) < 0 or bool((rank[kept] >= counts[idx[kept]]).any()):
            raise ValueError("slot rank outside [0, count of its expert)")
        key = idx[kept] * (int(rank.max()) + 1) + rank[kept]
        if key.unique().numel() != key.numel():
            raise ValueError("two slots of one expert share a rank")
    if offs is not None:
        offs = offs.reshape(-1).long().cpu()
        if bool((offs[1:] < offs[:-1]).any()) or int(offs[0]) != 0:
            raise ValueError("expert offsets are not a monotone prefix starting at 0")
        if capacity is not None and int(offs[-1]) > capacity:
            raise ValueError("expert offsets exceed the buffer: %d > %d" % (int(offs[-1]), capacity))


class EventTimer:
    r"""Accumulates CUDA-event durations of named regions on the current stream.

        timer = EventTimer()
        with timer("dispatch"):
            ...
        timer.summary(group)   # {"dispatch": {"ms": max over ranks, "calls": n}}
    """

    def __init__(self):
        self._pending = {}
        self._totals = {}

    @contextlib.contextmanager
    def __call__(self, name):
        if not torch.cuda.is_available():
            t0 = time.perf_counter()
            yield
            tot = self._totals.setdefault(name, [0.0, 0])
            tot[0] += (time.perf_counter() - t0) * 1e3
            tot[1] += 1
            return
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        with nvtx_range(name):
            yield
        end.record()
        self._pending.setdefault(name, []).append((start, end))

    def _flush(self):
        if self._pending:
            torch.cuda.synchronize()
        for name, pairs in self._pending.items():
            tot = self._totals.setdefault(name, [0.0, 0])
            for s, e in pairs:
                tot[0] += s.elapsed_time(e)
                tot[1] += 1
        self._pending.clear()

    def summary(self, group=None):
        self._flush()
        out = {}
        for name in sorted(self._totals):
            ms, calls = self._totals[name]
            if dist.is_available() and dist.is_initialized():
                dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
                t = torch.tensor([ms], dtype=torch.float64, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
                ms = float(t)
            out[name] = {"ms": ms, "calls": calls}
        return out

    def reset(self):
        self._pending.clear()
        self._totals.clear()


def roofline_fraction(flops, nvlink_bytes, seconds, peak_flops, link_bytes_per_s=770e9):
    r"""Achieved fraction of ``max(flops / peak_flops, nvlink_bytes / link_bandwidth)``."""
    bound = max(flops / peak_flops if peak_flops else 0.0,
                nvlink_bytes / link_bytes_per_s if link_bytes_per_s else 0.0)
    return bound / seconds if seconds > 0 else 0.0


class JsonlLogger:
    r"""Appends one JSON object per line (rank 0 only when a process group exists)."""

    def __init__(self, path):
        self.path = path

    def log(self, **fields):
        if dist.is_available() and dist.is_initialized() and dist.get_rank() != 0:
            return
        fields.setdefault("time", time.time())
        with open(self.path, "a") as f:
            f.write(json.dumps(fields) + "\n")
