r"""
Device-timed measurement of the expert-parallel layer and its exchange, one process per GPU.

    torchrun --nproc-per-node N --master-addr 127.0.0.1 bench/measure_exchange.py

For the headline layer shape (4096 tokens per GPU, top-2, d_model 1024, d_hidden 4096, 2 experts
per GPU, bf16, near-uniform routing) it times, with CUDA events and as the maximum over ranks:

* ``count_exchange``                         (counts to all peers, offsets from the full matrix)
* forward of the fused layer                 (count exchange, GEMM 1 with the dispatch fused in,
                                             GEMM 2 with the return push, combine)
* forward + backward of the fused layer
* the same layer on the collective-library path (``FMOE_FUSED=0``) for comparison
* one-shot all-reduce of a gate-gradient sized bucket

Every measured sequence starts right behind a tiny all-reduce on the same stream, which lines the
ranks up on the device (no host skew inside the measurement); the fused sequences are replayed
from a CUDA graph, as in training.  The script prints the roofline time of the forward — the
slower of FLOPs / measured GEMM peak and NVLink bytes / link bandwidth — and achieved / roofline.
"""
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from fastmoe_b200 import FMoETransformerMLP  # noqa: E402
from fastmoe_b200.ops import native  # noqa: E402
from fastmoe_b200.parallel import symm  # noqa: E402

LINK_BYTES_PER_S = 770e9       # measured peer-copy bandwidth per direction between two B200s (nominal 900e9)
GEMM_FLOPS = 1643.7e12         # measured burst cuBLAS bf16 rate of one B200


def main():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    world, rank = dist.get_world_size(), dist.get_rank()
    nat = native.get()
    n_tok, k, d, h, n_exp = 4096, 2, 1024, 4096, 2
    torch.manual_seed(1 + rank)
    layer = FMoETransformerMLP(num_expert=n_exp, d_model=d, d_hidden=h, world_size=world,
                               top_k=k).to(dev).to(torch.bfloat16)
    x = torch.randn(n_tok, d, device=dev, dtype=torch.bfloat16)
    gy = torch.randn(n_tok, d, device=dev, dtype=torch.bfloat16)
    gate_grad = torch.randn(n_exp * world * (d + 1), device=dev).to(torch.bfloat16)
    tiny = torch.zeros(64, device=dev, dtype=torch.float32)
    flush = torch.empty(64 * 1024 * 1024, dtype=torch.float32, device=dev)
    ws = symm.get_workspace(dist.group.WORLD, dev)
    assert ws is not None, "symmetric memory is not available"

    def align():
        symm.allreduce_flat(tiny, dist.group.WORLD)

    def fwd():
        with torch.no_grad():
            return layer(x)

    def fwd_bwd():
        layer.zero_grad(set_to_none=True)
        xx = x.detach().requires_grad_(True)
        layer(xx).backward(gy)

    def counts():
        lec, _r = nat.route(torch.randint(0, n_exp * world, (n_tok * k,), device=dev), n_exp * world)
        symm._Tables(ws, lec, n_exp, symm.receive_capacity(n_tok, k, world))  # pylint: disable=protected-access

    def allreduce():
        symm.allreduce_flat(gate_grad, dist.group.WORLD, 1.0 / world)

    def timed(fn, graph):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = None
        if graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
        samples = []
        for _ in range(15):
            flush.zero_()
            align()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            if g is not None:
                g.replay()
            else:
                fn()
            e.record()
            torch.cuda.synchronize()
            samples.append(s.elapsed_time(e) * 1e3)
        t = torch.tensor([statistics.median(samples)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    results = {"counts": timed(counts, False), "fused_fwd": timed(fwd, True),
               "fused_fwd_bwd": timed(fwd_bwd, True), "allreduce": timed(allreduce, False)}
    os.environ["FMOE_FUSED"] = "0"
    results["library_path_fwd"] = timed(fwd, False)
    results["library_path_fwd_bwd"] = timed(fwd_bwd, False)
    os.environ["FMOE_FUSED"] = "1"

    # phases inside the fused dispatch + GEMM kernel (eager launches, %globaltimer stamps)
    from fastmoe_b200.utils import profiling
    os.environ["FMOE_EP_TRACE"] = "1"
    for _ in range(5):
        flush.zero_()
        align()
        fwd()
    del os.environ["FMOE_EP_TRACE"]
    phases = profiling.ep_trace_summary()[-1]

    rows = n_tok * k                         # rows a rank receives on average
    remote_frac = (world - 1) / world
    link_bytes = 2 * rows * d * 2 * remote_frac            # dispatch + return, per direction the same
    flops_fwd = 2 * 2.0 * rows * d * h
    roof_fwd = max(flops_fwd / GEMM_FLOPS, link_bytes / LINK_BYTES_PER_S) * 1e6
    if rank == 0:
        print(json.dumps({"world": world, "us": results,
                          "roofline_fwd_us": roof_fwd,
                          "fused_fwd_over_roofline": roof_fwd / results["fused_fwd"],
                          "link_time_us": link_bytes / LINK_BYTES_PER_S * 1e6,
                          "dispatch_gemm_phases_rank0": phases,
                          "status": int(nat.read_status(local))}, indent=1))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
