r"""
Single-layer MoE MLP micro-benchmark with the reference harness's knobs.

Counterpart of ``tests/benchmark_mlp.py`` of the reference (``:83-140``): environment variables
``BATCH_SIZE`` (4096), ``D_MODEL`` (1024), ``D_HIDDEN`` (4096), ``NUM_EXPERT`` (64 per rank),
``TOP_K`` (2); 4 warm-up + 16 timed iterations of forward and backward; the same FLOP model
``2·(d·h·B·k·2 + B·d·E)`` per forward.  Unlike the reference, which reads ``time.time()`` without
synchronising the device, each phase is timed with CUDA events and the maximum over ranks is
reported.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _common import init_distributed, max_over_ranks  # noqa: E402

from fastmoe_b200 import FMoETransformerMLP  # noqa: E402


def main():
    rank, world, device = init_distributed()
    batch = int(os.environ.get("BATCH_SIZE", "4096"))
    d_model = int(os.environ.get("D_MODEL", "1024"))
    d_hidden = int(os.environ.get("D_HIDDEN", "4096"))
    n_exp = int(os.environ.get("NUM_EXPERT", "64"))
    top_k = int(os.environ.get("TOP_K", "2"))
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    torch.manual_seed(rank)
    moe = FMoETransformerMLP(num_expert=n_exp, d_model=d_model, d_hidden=d_hidden, world_size=world,
                             top_k=top_k).to(device).to(dtype)
    x = torch.randn(batch, d_model, device=device, dtype=dtype, requires_grad=True)
    fwd_ms, bwd_ms = [], []
    for it in range(20):
        if device.type == "cuda":
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ev[0].record()
            y = moe(x)
            ev[1].record()
            y.sum().backward()
            ev[2].record()
            torch.cuda.synchronize()
            f, b = ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2])
        else:
            import time
            t0 = time.perf_counter()
            y = moe(x)
            t1 = time.perf_counter()
            y.sum().backward()
            f, b = (t1 - t0) * 1e3, (time.perf_counter() - t1) * 1e3
        if it >= 4:
            fwd_ms.append(max_over_ranks(f, device))
            bwd_ms.append(max_over_ranks(b, device))
    gflop = 2 * (d_model * d_hidden * batch * top_k * 2 + batch * d_model * n_exp * world) / 1e9
    if rank == 0:
        mean = sum(fwd_ms) / len(fwd_ms)
        print("Time mean/max {:.3f}/{:.3f} ms fwd, back {:.3f} ms, {:.1f} GFLOP/s fwd per rank".format(
            mean, max(fwd_ms), sum(bwd_ms) / len(bwd_ms), gflop / mean * 1e3))


if __name__ == "__main__":
    main()
