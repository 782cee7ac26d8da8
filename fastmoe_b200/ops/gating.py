r"""
Gate math: top-k selection with softmax over the selected logits.

Parity: the ``topk`` → ``softmax`` sequence of ``fmoe/gates/naive_gate.py:31-38`` (ATen ops
in the reference).  On a GPU one kernel reads each logits row once, keeps the k largest in
registers, writes ids and probabilities, and a second small kernel applies the softmax
Jacobian in backward and scatters the result into the dense logits gradient.

``linear_topk_softmax`` goes one step further for the plain linear gate
(``fmoe/gates/naive_gate.py:24-38``: ``nn.Linear`` → ``topk`` → ``softmax``): with at most 64
experts the logits of a token fit in registers, so one kernel reads the token once and writes
logits, ids and probabilities, and the backward is two kernels (softmax Jacobian + ``dx``;
``dW`` and ``db``) instead of the six of the ATen sequence.
"""
import torch
from torch.autograd import Function

from . import native

MAX_FUSED_K = 8
MAX_FUSED_EXPERTS = 4096
MAX_SINGLE_PASS_EXPERTS = 8


def _topk_softmax_torch(logits, k):
    val, idx = torch.topk(logits, k=k, dim=-1, largest=True, sorted=True)
    return idx, torch.softmax(val, dim=-1)


class _TopkSoftmax(Function):
    @staticmethod
    def forward(ctx, logits, k):
        idx, score = native.get().gate_topk_softmax(logits.contiguous(), int(k))
        ctx.save_for_backward(idx, score)
        ctx.shape = logits.shape
        ctx.mark_non_differentiable(idx)
        return idx, score

    @staticmethod
    def backward(ctx, _grad_idx, grad_score):
        idx, score = ctx.saved_tensors
        grad_logits = native.get().gate_topk_softmax_bwd(
            grad_score.contiguous(), idx, score, int(ctx.shape[-1]))
        return grad_logits, None


def topk_softmax(logits, k):
    r"""``(idx int64 [B,k], prob [B,k])``: the k largest logits per row (descending) and their softmax."""
    if (logits.is_cuda and k <= MAX_FUSED_K and logits.shape[-1] <= MAX_FUSED_EXPERTS
            and logits.dtype in (torch.float32, torch.bfloat16, torch.float16)):
        return _TopkSoftmax.apply(logits, k)
    return _topk_softmax_torch(logits, k)


class _LinearTopkSoftmax(Function):
    r"""``logits = x W^T + b``, top-k ids and softmax of the selected logits as one op."""

    @staticmethod
    def forward(ctx, x, weight, bias, k):
        logits, idx, prob = native.get().gate_linear_topk(x, weight, bias, int(k))
        ctx.save_for_backward(x, weight, idx, prob)
        ctx.has_bias = bias is not None
        ctx.mark_non_differentiable(idx)
        ctx.set_materialize_grads(False)
        return logits, idx, prob

    @staticmethod
    def backward(ctx, grad_logits, _grad_idx, grad_prob):
        x, weight, idx, prob = ctx.saved_tensors
        if grad_logits is None and grad_prob is None:
            return None, None, None, None
        dx, dw, db, _dl = native.get().gate_linear_topk_bwd(
            None if grad_prob is None else grad_prob.contiguous(), idx, prob,
            None if grad_logits is None else grad_logits.contiguous(), x, weight,
            ctx.needs_input_grad[0], ctx.has_bias and ctx.needs_input_grad[2])
        return (dx if ctx.needs_input_grad[0] else None, dw if ctx.needs_input_grad[1] else None,
                db if ctx.has_bias and ctx.needs_input_grad[2] else None, None)


_PAD_BIAS = -30000.0   # bias of the padding columns: representable in bf16 and fp16, never selected
_OFFS_CACHE = {}


def _one_group_offs(rows, device):
    key = (rows, device)
    offs = _OFFS_CACHE.get(key)
    if offs is None:
        # built from device ops only, so that a first call inside a graph capture is legal
        offs = (torch.arange(2, device=device, dtype=torch.int32) * rows).contiguous()
        _OFFS_CACHE[key] = offs
    return offs


class _GateGemm(Function):
    r"""``logits = x W^T + b`` on the tcgen05 grouped-GEMM kernel (one group), for any number of
    experts.  The expert dimension is padded to a multiple of 64 — the padding columns get a
    large negative bias, so a top-k over the padded logits never selects them — and the
    backward products ``dx = dl W`` and ``dW = dl^T x`` (with ``db`` from the same launch) run on
    the same kernel's input-gradient and weight-gradient modes."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        from . import grouped_gemm as gg
        tot, d = weight.shape
        pad = (-tot) % 64
        wp = torch.nn.functional.pad(weight, (0, 0, 0, pad)).unsqueeze(0).contiguous()
        bp = torch.full((1, tot + pad), _PAD_BIAS, dtype=x.dtype, device=x.device)
        if bias is not None:
            bp[0, :tot] = bias
        else:
            bp[0, :tot] = 0
        offs = _one_group_offs(x.shape[0], x.device)
        logits = gg.forward(x, wp, offs, bp)
        ctx.save_for_backward(x, wp, offs)
        ctx.tot = tot
        ctx.has_bias = bias is not None
        return logits

    @staticmethod
    def backward(ctx, dl):
        from . import grouped_gemm as gg
        x, wp, offs = ctx.saved_tensors
        dl = dl.contiguous()
        dx = gg.dgrad(dl, wp, offs) if ctx.needs_input_grad[0] else None
        dw = db = None
        if ctx.needs_input_grad[1] or (ctx.has_bias and ctx.needs_input_grad[2]):
            dwp, dbp = gg.wgrad(dl, x, offs, 1, with_bias_grad=True)
            dw = dwp[0, :ctx.tot]
            db = dbp[0, :ctx.tot] if ctx.has_bias else None
        return dx, dw, db


def _gate_gemm_ok(x, weight, bias):
    from . import grouped_gemm as gg
    return (x.is_cuda and x.dim() == 2 and x.dtype in (torch.bfloat16, torch.float16)
            and weight.dtype == x.dtype and (bias is None or bias.dtype == x.dtype)
            and x.shape[1] % 64 == 0 and x.shape[0] > 0 and not torch.is_autocast_enabled()
            and native.available()
            and native.get().grouped_gemm_supported(gg.MODE_NT, 0, weight.shape[0] + (-weight.shape[0]) % 64,
                                                    x.shape[1], 1))


def linear_topk_softmax(x, weight, bias, k):
    r"""``(logits [B,E], idx int64 [B,k], prob [B,k])`` of a linear gate over 2-D ``x``.

    Uses the single-pass kernel when the shape allows it (16-bit types on a GPU, ``d_model`` a
    multiple of 8) and the expert count is small enough for its one-warp-per-token SIMT dot
    products to beat a library GEMM (measured on B200 with 4096 tokens, ``d_model`` 1024:
    30.6 vs 35.5 µs forward + backward at 2 experts, 52 vs 37 µs at 16).  Above that the
    product runs on the tcgen05 grouped-GEMM kernel with a single group (:class:`_GateGemm`),
    followed by :func:`topk_softmax`; only 32-/64-bit inputs, CPU tensors and odd ``d_model``
    take the ``linear`` → :func:`topk_softmax` sequence of PyTorch ops.
    """
    if (x.is_cuda and x.dim() == 2 and x.dtype in (torch.bfloat16, torch.float16)
            and weight.shape[0] <= MAX_SINGLE_PASS_EXPERTS
            and weight.dtype == x.dtype and (bias is None or bias.dtype == x.dtype)
            and not torch.is_autocast_enabled()
            and native.get().gate_fused_supported(weight.shape[0], x.shape[1], k)):
        xc = x if x.is_contiguous() else x.contiguous()
        return _LinearTopkSoftmax.apply(xc, weight.contiguous(), bias, k)
    if _gate_gemm_ok(x, weight, bias) and k <= MAX_FUSED_K:
        # more experts: tensor-core product on this library's own kernel, then the top-k /
        # softmax kernel over the (padded) logits
        tot = weight.shape[0]
        padded = _GateGemm.apply(x if x.is_contiguous() else x.contiguous(), weight, bias)
        idx, prob = topk_softmax(padded, k)
        return padded[:, :tot], idx, prob
    logits = torch.nn.functional.linear(x, weight, bias)
    idx, prob = topk_softmax(logits, k)
    return logits, idx, prob
