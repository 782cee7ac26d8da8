r"""
Small, self-terminating workloads for profiling single kernels under ``ncu``.

    python -m fastmoe_b200.ops.profile_cases gemm      # the six grouped-GEMM variants of one MoE layer
    python -m fastmoe_b200.ops.profile_cases rows      # routing / scatter / combine kernels
    python -m fastmoe_b200.ops.profile_cases push      # exchange kernels on one GPU (one-rank group)
    python -m fastmoe_b200.ops.profile_cases push_gemm # GEMM 2 with the return push in its epilogue (one-rank group)
    python -m fastmoe_b200.ops.profile_cases gate      # single-pass linear gate, forward and backward

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
        gg.wgrad(hid, x, offs, n_exp, with_bias_grad=True)       # wgrad 1 (+ bias gradient)
        gg.wgrad(x, hid, offs, n_exp, with_bias_grad=True)       # wgrad 2 (+ bias gradient)
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


def push_case(repeats=3):
    r"""The sender / receiver kernels of the expert-parallel exchange in a one-rank process
    group: every row is "sent" to this GPU's own symmetric buffer, so the kernels run exactly
    the code of the multi-GPU path (peer tables, flags, fences) without a second GPU."""
    import os
    import torch.distributed as dist
    from ..parallel import symm
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    nat = native.get()
    ws = symm.get_workspace(dist.group.WORLD, dev)
    assert ws is not None, "symmetric memory is not available"
    n_tok, k, d, n_exp = 4096, 2, 1024, 2
    x = torch.randn(n_tok, d, device=dev, dtype=torch.bfloat16)
    idx = torch.randint(0, n_exp, (n_tok * k,), device=dev)
    score = torch.rand(n_tok * k, device=dev).to(torch.bfloat16)
    capacity = symm.receive_capacity(n_tok, k, 1)
    rows_buf, rows_ptrs = ws.buffer("rows", capacity * d * 2)
    meta_buf, meta_ptrs = ws.buffer("meta", capacity * 8)
    ret_buf, ret_ptrs = ws.buffer("ret", n_tok * k * d * 2)
    lec, rnk = nat.route(idx, n_exp)
    dst_base = torch.empty(n_exp, dtype=torch.int32, device=dev)
    offs = torch.empty(n_exp + 1, dtype=torch.int32, device=dev)
    total = torch.empty(1, dtype=torch.int32, device=dev)
    xs = torch.empty(capacity, d, device=dev, dtype=torch.bfloat16)
    meta = torch.empty(capacity, dtype=torch.int64, device=dev)
    out = torch.empty(n_tok, d, device=dev, dtype=torch.bfloat16)
    keep = torch.empty(n_tok * k, d, device=dev, dtype=torch.bfloat16)
    for _ in range(repeats):
        ws.ctx.count_exchange(lec, ws.cnt_ptrs, n_exp, capacity, dst_base, offs, total)
        ws.ctx.begin_epoch()
        ws.ctx.dispatch_push(x, idx, rnk, dst_base, None, rows_ptrs, meta_ptrs, n_exp, k, capacity)
        ws.ctx.wait_copy(nat.P2P_CHAN_DISPATCH, rows_buf, meta_buf.view(torch.int64), total, xs, meta)
        ws.ctx.return_push(xs, meta, total, ret_ptrs)
        ws.ctx.wait_combine(ret_buf, idx, score, k, out, keep)
    torch.cuda.synchronize()
    assert nat.read_status(0) == 0
    # every token came back as the score-weighted sum of its own k copies
    want = x.float() * score.float().view(n_tok, k).sum(1, keepdim=True)
    assert torch.allclose(out.float(), want, atol=0.05, rtol=0.05)
    dist.destroy_process_group()


def push_gemm_case(repeats=3):
    r"""The fused combine on one GPU: the second expert GEMM whose epilogue stores every output
    row into the slot-indexed return buffer (here this rank's own symmetric buffer, reached
    through the same peer table, completion counter and flags as on several GPUs), followed by
    the gate-weighted combine.  Checked against the plain GEMM + local combine."""
    import os
    import torch.distributed as dist
    from ..parallel import symm
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29578")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    nat = native.get()
    ws = symm.get_workspace(dist.group.WORLD, dev)
    assert ws is not None, "symmetric memory is not available"
    n_tok, k, d, h, n_exp = 4096, 2, 1024, 4096, 2
    x = torch.randn(n_tok, d, device=dev, dtype=torch.bfloat16)
    idx = torch.randint(0, n_exp, (n_tok * k,), device=dev)
    score = torch.rand(n_tok * k, device=dev).to(torch.bfloat16)
    w2 = (torch.randn(n_exp, d, h, device=dev) * 0.02).to(torch.bfloat16)
    b2 = (torch.randn(n_exp, d, device=dev) * 0.1).to(torch.bfloat16)
    capacity = symm.receive_capacity(n_tok, k, 1)
    act = torch.randn(capacity, h, device=dev, dtype=torch.bfloat16)
    rows_buf, rows_ptrs = ws.buffer("rows", capacity * d * 2)
    meta_buf, meta_ptrs = ws.buffer("meta", capacity * 8)
    ret_buf, ret_ptrs = ws.buffer("ret", n_tok * k * d * 2)
    lec, rnk = nat.route(idx, n_exp)
    dst_base = torch.empty(n_exp, dtype=torch.int32, device=dev)
    offs = torch.empty(n_exp + 1, dtype=torch.int32, device=dev)
    total = torch.empty(1, dtype=torch.int32, device=dev)
    xs = torch.empty(capacity, d, device=dev, dtype=torch.bfloat16)
    meta = torch.empty(capacity, dtype=torch.int64, device=dev)
    out = torch.empty(n_tok, d, device=dev, dtype=torch.bfloat16)
    keep = torch.empty(n_tok * k, d, device=dev, dtype=torch.bfloat16)
    for _ in range(repeats):
        ws.ctx.count_exchange(lec, ws.cnt_ptrs, n_exp, capacity, dst_base, offs, total)
        ws.ctx.begin_epoch()
        ws.ctx.dispatch_push(x, idx, rnk, dst_base, None, rows_ptrs, meta_ptrs, n_exp, k, capacity)
        ws.ctx.wait_copy(nat.P2P_CHAN_DISPATCH, rows_buf, meta_buf.view(torch.int64), total, xs, meta)
        ws.ctx.gemm_push(gg.MODE_NT, act, w2, offs, b2, meta, ret_ptrs)
        ws.ctx.wait_combine(ret_buf, idx, score, k, out, keep)
    torch.cuda.synchronize()
    assert nat.read_status(0) == 0
    ys = gg.forward(act, w2, offs, b2)
    want = torch.empty_like(out)
    nat.gather_combine(ys, idx, rnk, offs[:n_exp].contiguous(), score, k, want)
    assert torch.allclose(out.float(), want.float(), atol=0.05, rtol=0.05)
    dist.destroy_process_group()


def gate_case(repeats=3):
    from . import gating
    dev = "cuda"
    n_tok, d, tot, k = 32768, 1024, 8, 2
    x = torch.randn(n_tok, d, device=dev, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(tot, d, device=dev) * 0.03).to(torch.bfloat16).requires_grad_(True)
    b = torch.zeros(tot, device=dev, dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(n_tok, k, device=dev, dtype=torch.bfloat16)
    for _ in range(repeats):
        _logits, _idx, prob = gating.linear_topk_softmax(x, w, b, k)
        prob.backward(g)
    torch.cuda.synchronize()


if __name__ == "__main__":
    {"gemm": gemm_case, "rows": rows_case, "push": push_case, "push_gemm": push_gemm_case,
     "gate": gate_case}[sys.argv[1] if len(sys.argv) > 1 else "gemm"]()
    print("done")
