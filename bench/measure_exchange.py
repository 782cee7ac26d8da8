r"""
Device-timed measurement of the peer-to-peer exchange paths, one process per GPU.

    torchrun --nproc-per-node N --master-addr 127.0.0.1 -m fastmoe_b200.parallel.measure_exchange

For the headline layer shape (4096 tokens per GPU, top-2, d_model 1024, d_hidden 4096, 2 experts
per GPU, bf16, near-uniform routing) it times, with CUDA events and as the maximum over ranks:

* ``count_exchange``                         (counts to all peers, offsets from the full matrix)
* ``dispatch_push`` + ``wait_copy``          (rows to the owners, arrival, copy out of staging)
* local GEMM 2                               (for comparison)
* ``gemm_push`` + ``wait_combine``           (GEMM 2 whose epilogue returns rows to the sources,
                                             arrival, gate-weighted combine)
* one-shot all-reduce of the gate gradients

Each measured sequence starts right behind a tiny all-reduce on the same stream, which lines
the ranks up on the device (no host skew inside the measurement).  For every path the script
prints the roofline time — the slower of FLOPs / measured GEMM peak and NVLink bytes / link
bandwidth — and achieved / roofline.
"""
import json
import os
import statistics

import torch
import torch.distributed as dist

from ..ops import grouped_gemm as gg
from ..ops import native
from . import symm

LINK_BYTES_PER_S = 770e9       # measured peer-copy bandwidth per direction between two B200s (nominal 900e9)
GEMM_FLOPS = 1643.7e12         # measured burst cuBLAS bf16 rate of one B200


def main():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    world, rank = dist.get_world_size(), dist.get_rank()
    nat = native.get()
    ws = symm.get_workspace(dist.group.WORLD, dev)
    assert ws is not None, "symmetric memory is not available"

    n_tok, k, d, h, n_exp = 4096, 2, 1024, 4096, 2
    tot = n_exp * world
    torch.manual_seed(1 + rank)
    x = torch.randn(n_tok, d, device=dev, dtype=torch.bfloat16)
    idx = torch.randint(0, tot, (n_tok * k,), device=dev)
    score = torch.rand(n_tok * k, device=dev).to(torch.bfloat16)
    w2 = (torch.randn(n_exp, d, h, device=dev) * 0.02).to(torch.bfloat16)
    b2 = torch.zeros(n_exp, d, device=dev, dtype=torch.bfloat16)
    gate_grad = torch.randn(tot * d + tot, device=dev).to(torch.bfloat16)
    capacity = symm.receive_capacity(n_tok, k, world)

    lec, rnk = nat.route(idx, tot)
    dst_base = torch.empty(tot, dtype=torch.int32, device=dev)
    offs = torch.empty(n_exp + 1, dtype=torch.int32, device=dev)
    total = torch.empty(1, dtype=torch.int32, device=dev)
    rows_buf, rows_ptrs = ws.buffer("rows", capacity * d * 2)
    meta_buf, meta_ptrs = ws.buffer("meta", capacity * 8)
    ret_buf, ret_ptrs = ws.buffer("ret", n_tok * k * d * 2)
    xs = torch.empty(capacity, d, device=dev, dtype=torch.bfloat16)
    meta = torch.empty(capacity, dtype=torch.int64, device=dev)
    act = torch.randn(capacity, h, device=dev, dtype=torch.bfloat16)
    out = torch.empty(n_tok, d, device=dev, dtype=torch.bfloat16)
    keep = torch.empty(n_tok * k, d, device=dev, dtype=torch.bfloat16)
    tiny = torch.zeros(64, device=dev, dtype=torch.float32)

    def align():
        symm.allreduce_flat(tiny, dist.group.WORLD)

    def counts():
        ws.ctx.count_exchange(lec, ws.cnt_ptrs, n_exp, capacity, dst_base, offs, total)

    def dispatch():
        ws.ctx.dispatch_push(x, idx, rnk, dst_base, None, rows_ptrs, meta_ptrs, n_exp, k, capacity)
        ws.ctx.wait_copy(nat.P2P_CHAN_DISPATCH, rows_buf, meta_buf.view(torch.int64), total, xs, meta)

    def gemm_local():
        gg.forward(act, w2, offs, b2)

    def gemm_push_combine():
        ws.ctx.gemm_push(gg.MODE_NT, act, w2, offs, b2, meta, ret_ptrs)
        ws.ctx.wait_combine(ret_buf, idx, score, k, out, keep)

    def allreduce():
        symm.allreduce_flat(gate_grad, dist.group.WORLD, 1.0 / world)

    def exchange_round(timed):
        # one full, consistent exchange; `timed` selects which part sits between the events
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        align()
        if timed == "counts":
            s.record(); counts(); e.record()
        else:
            counts()
        if timed == "dispatch":
            align(); s.record(); dispatch(); e.record()
        else:
            dispatch()
        if timed == "gemm_local":
            align(); s.record(); gemm_local(); e.record()
        if timed == "gemm_push":
            align(); s.record(); gemm_push_combine(); e.record()
        else:
            gemm_push_combine()
        if timed == "allreduce":
            align(); s.record(); allreduce(); e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) * 1e3  # microseconds

    results = {}
    for name in ("counts", "dispatch", "gemm_local", "gemm_push", "allreduce"):
        for _ in range(3):
            exchange_round(name)
        samples = [exchange_round(name) for _ in range(15)]
        t = torch.tensor([statistics.median(samples)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        results[name] = float(t)

    rows_recv = int(total.item())
    remote_frac = (world - 1) / world
    row_bytes = n_tok * k * d * 2 * remote_frac
    flops2 = 2.0 * rows_recv * d * h
    roof = {
        "dispatch": row_bytes / LINK_BYTES_PER_S * 1e6,
        "gemm_local": flops2 / GEMM_FLOPS * 1e6,
        "gemm_push": max(flops2 / GEMM_FLOPS, row_bytes / LINK_BYTES_PER_S) * 1e6,
    }
    if rank == 0:
        report = {"world": world, "rows_received_rank0": rows_recv, "us": results,
                  "roofline_us": roof,
                  "achieved_over_roofline": {k2: roof[k2] / results[k2] for k2 in roof},
                  "status": int(nat.read_status(local))}
        print(json.dumps(report, indent=1))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
