r"""
Python front-end of the grouped GEMM kernels.

The three products of a grouped linear — forward ``Y_e = X_e W_e^T (+b_e)``, input gradient
``dX_e = dY_e W_e`` and weight gradient ``dW_e = dY_e^T X_e`` (``cuda/parallel_linear.cuh:74-84,
124-147`` in the reference, one cuBLAS call each per expert) — are single launches of the
tcgen05 kernel for bf16/fp16 with tensor-core-friendly shapes, and of the reference-precision
SIMT kernel for fp32/fp64 or odd shapes.  Row offsets are an int32 device tensor
``offs[E+1]``; only the compatibility entry points below take host counts.
"""
import torch

from . import native

MODE_NT, MODE_NN, MODE_WGRAD = 0, 1, 2
ACT_CODES = {None: 0, "identity": 0, "relu": 1, "gelu": 2, "gelu_tanh": 3}
EPI_BIAS_ACT, EPI_DACT = 0, 1

_TC = (torch.bfloat16, torch.float16)


def offsets_from_counts(counts, device):
    r"""int32 ``[E+1]`` exclusive prefix of host-resident ``counts``, placed on ``device``."""
    c = torch.as_tensor(counts).reshape(-1).to(torch.int64)
    offs = torch.zeros(c.numel() + 1, dtype=torch.int32)
    offs[1:] = torch.cumsum(c, 0).to(torch.int32)
    return offs.to(device, non_blocking=True)


def _tc_ok(t, mode, m, n, k, groups):
    return t.dtype in _TC and native.get().grouped_gemm_supported(mode, m, n, k, groups)


def _aligned(t):
    r"""The tensor-core kernel wants 32-byte aligned, contiguous operands.  Views into flat
    buffers (e.g. the replicas ``nn.DataParallel`` broadcasts) may not be: copy those."""
    if t is None:
        return None
    if not t.is_contiguous() or t.data_ptr() % 32 != 0:
        return t.contiguous().clone() if t.data_ptr() % 32 != 0 and t.is_contiguous() else t.contiguous()
    return t


TILE_M, TILE_N = 128, 256


def pre_buffer(rows_cap, n, groups, dtype, device):
    r"""Storage of the saved pre-activation of a fused first GEMM: one ``128 x 256`` block per
    output tile, in the tile-blocked order the tensor-core epilogues write and read it (a 1-D
    tensor; :func:`untile_pre` gives the ``[rows, n]`` view of it for inspection)."""
    tiles = ((rows_cap + TILE_M - 1) // TILE_M + groups) * ((n + TILE_N - 1) // TILE_N)
    return torch.empty(tiles * TILE_M * TILE_N, dtype=dtype, device=device)


def untile_pre(pre, offs, n, rows_cap):
    r"""``[rows_cap, n]`` row-major copy of a tile-blocked pre-activation (rows outside the
    expert segments are zero).  For tests and debugging: reads ``offs`` on the host."""
    o = [int(v) for v in offs.tolist()]
    n_tiles = (n + TILE_N - 1) // TILE_N
    out = torch.zeros(rows_cap, n, dtype=pre.dtype, device=pre.device)
    blocks = pre.view(-1, 8, 4, 4, 32, 8)      # tile, warp (half*4 + part), chunk, piece, lane, 8 values
    tile = 0
    for e in range(len(o) - 1):
        rows = o[e + 1] - o[e]
        for m in range((rows + TILE_M - 1) // TILE_M):
            for nt in range(n_tiles):
                blk = blocks[tile]                                    # [8, 4, 4, 32, 8]
                blk = blk.view(2, 4, 4, 4, 32, 8)                      # half, part, chunk, piece, lane, v
                full = blk.permute(1, 4, 0, 2, 3, 5).reshape(TILE_M, TILE_N)   # (part, lane) x (half, chunk, piece, v)
                r0, c0 = o[e] + m * TILE_M, nt * TILE_N
                nr, nc = min(TILE_M, o[e + 1] - r0), min(TILE_N, n - c0)
                out[r0:r0 + nr, c0:c0 + nc] = full[:nr, :nc]
                tile += 1
    return out


def forward(x, weight, offs, bias=None, act=None, want_pre=False):
    r"""``act(x W^T + b)`` per expert; optionally also the pre-activation (for backward).

    On the tensor-core path with a fused activation the pre-activation comes back tile-blocked
    (1-D, see :func:`pre_buffer`); hand it to :func:`dgrad` as it is."""
    nat = native.get()
    groups, n, k = weight.shape
    out = torch.empty(x.shape[0], n, dtype=x.dtype, device=x.device)
    pre = None
    code = ACT_CODES[act]
    if x.shape[0] == 0:
        return (out, out.clone()) if want_pre else out
    if _tc_ok(x, MODE_NT, 0, n, k, groups):
        if want_pre and code != 0:
            pre = pre_buffer(x.shape[0], n, groups, x.dtype, x.device)
        nat.grouped_gemm(MODE_NT, _aligned(x), _aligned(weight), offs, out, _aligned(bias), pre, None,
                         code, EPI_BIAS_ACT, False)
        if want_pre and pre is None:
            pre = out
    else:
        nat.simt_grouped_gemm(MODE_NT, x, weight, offs, out, bias)
        _zero_tail(out, offs)
        if want_pre:
            pre = out
        if code != 0:
            out = _torch_act(out, act)
    return (out, pre) if want_pre else out


def dgrad(dy, weight, offs, pre=None, act=None):
    r"""``(dy W) * act'(pre)`` per expert (``pre`` = saved pre-activation of the producing layer,
    tile-blocked as :func:`forward` returned it, or a plain ``[rows, n]`` matrix)."""
    nat = native.get()
    groups, k, n = weight.shape
    out = torch.empty(dy.shape[0], n, dtype=dy.dtype, device=dy.device)
    code = ACT_CODES[act] if pre is not None else 0
    if dy.shape[0] == 0:
        return out
    if _tc_ok(dy, MODE_NN, 0, n, k, groups) and (not code or pre.dim() == 1):
        nat.grouped_gemm(MODE_NN, _aligned(dy), _aligned(weight), offs, out, None, None,
                         pre if code else None, code, EPI_DACT if code else EPI_BIAS_ACT, False)
    elif _tc_ok(dy, MODE_NN, 0, n, k, groups):
        # a row-major pre-activation: plain tensor-core product, derivative as a PyTorch op
        nat.grouped_gemm(MODE_NN, _aligned(dy), _aligned(weight), offs, out, None, None, None, 0,
                         EPI_BIAS_ACT, False)
        _zero_tail(out, offs)
        out = out * _torch_act_grad(pre, act)
    else:
        nat.simt_grouped_gemm(MODE_NN, dy, weight, offs, out, None)
        _zero_tail(out, offs)
        if code:
            out = out * _torch_act_grad(pre, act)
    return out


def wgrad(dy, x, offs, groups, out=None, accumulate=False, with_bias_grad=False):
    r"""``dW[e] = dy[rows_e]^T x[rows_e]`` → ``[E, dy.shape[1], x.shape[1]]``; empty experts give zeros.

    With ``with_bias_grad`` the per-expert column sums of ``dy`` (the bias gradient of the same
    grouped linear, ``[E, dy.shape[1]]``) are returned as well: ``(dW, db)``.  The tensor-core
    kernel produces them from the ``dy`` tiles it stages in shared memory anyway, so they cost
    no extra pass over ``dy`` and no extra launch.
    """
    nat = native.get()
    m, n = dy.shape[1], x.shape[1]
    if out is None:
        out = torch.empty(groups, m, n, dtype=dy.dtype, device=dy.device)
        accumulate = False
    db = None
    if _tc_ok(dy, MODE_WGRAD, m, n, 0, groups) and out.data_ptr() % 32 == 0:
        if with_bias_grad:
            db = torch.empty(groups, m, dtype=dy.dtype, device=dy.device)
        nat.grouped_gemm(MODE_WGRAD, _aligned(dy), _aligned(x), offs, out, None, None, None, 0, 0,
                         accumulate, db)
    else:
        tmp = torch.empty(groups, m, n, dtype=dy.dtype, device=dy.device)
        nat.simt_grouped_gemm(MODE_WGRAD, dy, x, offs, tmp, None)
        if accumulate:
            out += tmp
        else:
            out.copy_(tmp)
        if with_bias_grad:
            db = bias_grad(dy, offs)
    return (out, db) if with_bias_grad else out


def bias_grad(dy, offs, dtype=None):
    r"""Column sums of ``dy`` per expert → ``[E, n]`` (fp32 accumulation)."""
    if dy.dtype in _TC and dy.shape[1] % 8 == 0:
        out = native.get().colsum(dy, offs)
    else:
        groups = offs.numel() - 1
        rows = torch.arange(dy.shape[0], device=dy.device)
        seg = torch.bucketize(rows, offs[1:].long(), right=True)
        valid = rows < offs[-1].long()
        out = torch.zeros(groups + 1, dy.shape[1], dtype=torch.float64 if dy.dtype == torch.float64
                          else torch.float32, device=dy.device)
        out.index_add_(0, torch.where(valid, seg, torch.full_like(seg, groups)), dy.to(out.dtype))
        out = out[:groups]
    return out.to(dtype if dtype is not None else dy.dtype)


def _zero_tail(out, offs):
    r"""The SIMT kernel leaves rows past the last expert segment unwritten (the buffer comes from
    ``torch.empty``): zero them, without a host read, so that an activation applied to the whole
    buffer never meets NaN bit patterns."""
    rows = torch.arange(out.shape[0], device=out.device)
    out.masked_fill_((rows >= offs[-1])[:, None], 0)


def _torch_act(x, act):
    if act == "relu":
        return torch.relu(x)
    if act == "gelu":
        return torch.nn.functional.gelu(x)
    if act == "gelu_tanh":
        return torch.nn.functional.gelu(x, approximate="tanh")
    return x


def _torch_act_grad(pre, act):
    x = pre.detach().clone().requires_grad_(True)
    with torch.enable_grad():
        y = _torch_act(x, act)
    (g,) = torch.autograd.grad(y, x, torch.ones_like(y))
    return g


# ----------------------------------------------------------------------------------------
# Compatibility entry points: host-resident counts (the reference's calling convention).
# ----------------------------------------------------------------------------------------
def linear_forward_host_counts(inp, expert_count_cpu, weight, bias=None):
    offs = offsets_from_counts(expert_count_cpu, inp.device)
    return forward(inp.contiguous(), weight.contiguous(), offs,
                   bias.contiguous() if bias is not None else None)


def linear_backward_host_counts(grad_out, inp, expert_count_cpu, weight, bias=None):
    offs = offsets_from_counts(expert_count_cpu, inp.device)
    grad_out = grad_out.contiguous()
    grad_in = dgrad(grad_out, weight.contiguous(), offs)
    if bias is not None:
        grad_w, grad_b = wgrad(grad_out, inp.contiguous(), offs, weight.shape[0], with_bias_grad=True)
        grad_b = grad_b.to(bias.dtype)
    else:
        grad_w, grad_b = wgrad(grad_out, inp.contiguous(), offs, weight.shape[0]), None
    return grad_in, grad_w, grad_b
