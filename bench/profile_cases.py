r"""
Small, self-terminating workloads for profiling single kernels under ``ncu``.

    python bench/profile_cases.py gemm      # the six grouped-GEMM variants of one MoE layer
    python bench/profile_cases.py rows      # routing / scatter / combine kernels
    python bench/profile_cases.py ep_layer  # fused expert-parallel layer, fwd + bwd, in a one-rank group
    python bench/profile_cases.py gate      # single-pass linear gate, forward and backward

Each case touches more than the 126 MB L2 in total but holds well under 1 GB on the device and
launches each kernel a handful of times, so that a full-metric capture of two or three launches
ends by itself within a minute.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from fastmoe_b200.ops import grouped_gemm as gg  # noqa: E402
from fastmoe_b200.ops import native  # noqa: E402


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
    pre = gg.pre_buffer(rows, h, n_exp, torch.bfloat16, dev).normal_()   # tile-blocked pre-activation
    for _ in range(repeats):
        gg.forward(x, w1, offs, b1, act="gelu", want_pre=True)   # GEMM 1: NT + bias + GELU + pre-activation
        gg.forward(hid, w2, offs, None)                          # GEMM 2: NT plain
        gg.dgrad(x, w2, offs, pre=pre, act="gelu")               # dgrad 2: NN + GELU derivative
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


def _one_rank_group(port):
    import os
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", str(port))
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    return dev


def ep_layer_case(repeats=3, n_tok=4096, d=1024, h=4096, n_exp=2, k=2):
    r"""The fused expert-parallel layer in a one-rank process group: every row is "sent" to this
    GPU's own symmetric buffers, so the kernels run exactly the code of the multi-GPU path
    (sender warps and arrival-gated tiles in the first GEMM launch, return push in the epilogue
    of the second, peer tables, flags, fences) without a second GPU.  Checked against the
    single-GPU fused path of the same layer."""
    import torch.distributed as dist
    from fastmoe_b200 import FMoETransformerMLP
    from fastmoe_b200.ops import fused
    from fastmoe_b200.parallel import symm
    dev = _one_rank_group(29577)
    torch.manual_seed(0)
    layer = FMoETransformerMLP(num_expert=n_exp, d_model=d, d_hidden=h, top_k=k).to(dev).to(torch.bfloat16)
    x = torch.randn(n_tok, d, device=dev, dtype=torch.bfloat16)
    gy = torch.randn(n_tok, d, device=dev, dtype=torch.bfloat16)
    with torch.no_grad():
        idx, score = layer.gate(x)

    def run(fn):
        layer.zero_grad()
        xx = x.clone().requires_grad_(True)
        sc = score.clone().requires_grad_(True)
        y = fn(layer, xx, idx, sc)
        y.backward(gy)
        return y.float(), xx.grad.float(), sc.grad.float(), layer.experts.htoh4.weight.grad.float().clone()

    for _ in range(repeats):
        got = run(symm.moe_mlp_forward)
    torch.cuda.synchronize()
    assert native.get().read_status(0) == 0, native.get().read_status(0)
    want = run(fused.moe_mlp_forward)
    for g, w in zip(got, want):
        err = float((g - w).abs().max())
        assert err <= 0.05 * float(w.abs().max()) + 1e-2, err
    # device time of every grouped-GEMM launch of the two paths (fused dispatch / return push
    # against the plain single-GPU kernels)
    from torch.profiler import ProfilerActivity, profile
    for name, fn in (("expert-parallel kernels", symm.moe_mlp_forward), ("single-GPU path", fused.moe_mlp_forward)):
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(5):
                run(fn)
            torch.cuda.synchronize()
        for ev in sorted(prof.key_averages(), key=lambda e: e.key):
            if "grouped_gemm" in ev.key or "scatter" in ev.key or "combine" in ev.key:
                print("%-24s %-58s %8.1f us x %d" % (name, ev.key[:58], ev.device_time_total / ev.count,
                                                     ev.count // 5))
    dist.destroy_process_group()


def gate_case(repeats=3):
    from fastmoe_b200.ops import gating
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
    {"gemm": gemm_case, "rows": rows_case, "ep_layer": ep_layer_case,
     "gate": gate_case}[sys.argv[1] if len(sys.argv) > 1 else "gemm"]()
    print("done")
