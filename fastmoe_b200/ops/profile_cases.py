r"""
Small, self-terminating workloads for profiling single kernels under ``ncu``.

    python -m fastmoe_b200.ops.profile_cases gemm      # the six grouped-GEMM variants of one MoE layer
    python -m fastmoe_b200.ops.profile_cases rows      # routing / scatter / combine kernels

Each case touches more than the 126 MB L2 in total but holds well under 1 GB on the device and
launches each kernel a handful of times, so that a full-metric capture of two or three launches
ends by itself within a minute.
"""
import sys

import torch

from . import grouped_gemm as gg
from . import native


def gemm_case(repeats=2):
    dev = "cuda"
    n_exp, rows_per, d, h = 2, 4096, 1024, 4096
    rows = n_exp * rows_per
    x = torch.randn(rows, d, device=dev, dtype=torch.bfloat16)
    w1 = torch.randn(n_exp, h, d, device=dev, dtype=torch.bfloat16) * 0.02
    b1 = torch.zeros(n_exp, h, device=dev, dtype=torch.bfloat16)
    w2 = torch.randn(n_exp, d, h, device=dev, dtype=torch.bfloat16) * 0.02
    offs = torch.arange(0, rows + 1, rows_per, device=dev, dtype=torch.int32)
    hid = torch.randn(rows, h, device=dev, dtype=torch.bfloat16)
    for _ in range(repeats):
        gg.forward(x, w1, offs, b1, act="gelu", want_pre=True)   # GEMM 1: NT + bias + GELU + pre-activation
        gg.forward(hid, w2, offs, None)                          # GEMM 2: NT plain
        gg.dgrad(x, w2, offs, pre=hid, act="gelu")               # dgrad 2: NN + GELU derivative
        gg.dgrad(hid, w1, offs)                                  # dgrad 1: NN plain
        gg.wgrad(hid, x, offs, n_exp)                            # wgrad 1
        gg.wgrad(x, hid, offs, n_exp)                            # wgrad 2
    torch.cuda.synchronize()
    assert native.get().read_status(0) == 0


def rows_case(repeats=2):
    nat = native.get()
    dev = "cuda"
    n_tok, k, d, tot = 32768, 2, 1024, 16
    x = torch.randn(n_tok, d, device=dev, dtype=torch.bfloat16)
    idx = torch.randint(0, tot, (n_tok * k,), device=dev)
    score = torch.rand(n_tok * k, device=dev).to(torch.bfloat16)
    rows = torch.empty(n_tok * k, d, device=dev, dtype=torch.bfloat16)
    out = torch.empty(n_tok, d, device=dev, dtype=torch.bfloat16)
    for _ in range(repeats):
        _counts, rank, offs = nat.route_offs(idx, tot)
        nat.scatter_rows(x, idx, rank, offs, None, k, rows, None)
        nat.gather_combine(rows, idx, rank, offs, score, k, out)
        nat.colsum(rows, offs)
    torch.cuda.synchronize()


if __name__ == "__main__":
    {"gemm": gemm_case, "rows": rows_case}[sys.argv[1] if len(sys.argv) > 1 else "gemm"]()
    print("done")
