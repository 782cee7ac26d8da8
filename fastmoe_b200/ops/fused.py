r"""
The fused device path of ``FMoETransformerMLP``.

One layer call is a fixed sequence of kernels with no host read in between:

    route (count + rank + offsets)  →  dispatch (rows to expert segments; peer-to-peer stores
    when the experts live on other GPUs)  →  grouped GEMM 1 (+bias, +activation, pre-activation
    kept)  →  grouped GEMM 2 (+bias)  →  combine (gate-weighted sum of the top-k rows)

It replaces ``_fmoe_general_global_forward`` of the reference (``fmoe/layers.py:26-78``:
``prepare_forward`` with two host syncs, ``MOEScatter``, a Python loop over experts with two
synchronising linears each, ``MOEGather``, ``bmm``).  Buffers are sized from host-known
quantities only (``B·k`` rows on one GPU, the configured receive capacity on several), so
autograd never needs a count on the host.  Backward mirrors forward: the combine backward
produces ``d score`` and the scaled output gradients in one pass, the activation derivative
is applied in the epilogue of the input-gradient GEMM, and the weight gradients reduce over
token rows on the tensor cores.
"""
import torch
from torch.autograd import Function

from . import grouped_gemm as gg
from . import native
from .. import config
from ..transformer import activation_kind
from ..utils.profiling import check_routing, fused_range

_TC = (torch.bfloat16, torch.float16)


def supports(layer, x, idx):
    r"""Whether the fused kernels can run this call (else the general path is used)."""
    if not native.available() or x.dtype not in _TC or idx.dim() != 2:
        return False
    e = layer.experts
    if e.htoh4.weight.dtype != x.dtype or e.htoh4.bias is None or e.h4toh.bias is None:
        return False
    d, h = layer.d_model, layer.d_hidden
    if d % 64 != 0 or h % 64 != 0:
        return False
    if layer.world_size > 1 or _forced_ep():
        from ..parallel import symm
        return symm.fused_available(layer, x)
    return True


def _forced_ep():
    if not config.force_ep_path():
        return False
    import torch.distributed as dist
    return dist.is_available() and dist.is_initialized()


class _Dispatch(Function):
    r"""``xs[offs[e] + rank[s]] = x[s // k]`` for every kept slot ``s`` routed to expert ``e``."""

    @staticmethod
    def forward(ctx, x, idx, rank, offs, k):
        nat = native.get()
        xs = torch.empty(idx.numel(), x.shape[1], dtype=x.dtype, device=x.device)
        nat.scatter_rows(x, idx, rank, offs, None, k, xs, None)
        ctx.save_for_backward(idx, rank, offs)
        ctx.k = k
        ctx.n_tok = x.shape[0]
        return xs

    @staticmethod
    def backward(ctx, dxs):
        idx, rank, offs = ctx.saved_tensors
        dx = torch.empty(ctx.n_tok, dxs.shape[1], dtype=dxs.dtype, device=dxs.device)
        native.get().gather_combine(dxs.contiguous(), idx, rank, offs, None, ctx.k, dx)
        return dx, None, None, None, None


class _Combine(Function):
    r"""``out[t] = Σ_j score[t, j] · ys[row(t, j)]``; dropped slots contribute nothing."""

    @staticmethod
    def forward(ctx, ys, score, idx, rank, offs, k):
        n_tok = idx.numel() // k
        out = torch.empty(n_tok, ys.shape[1], dtype=ys.dtype, device=ys.device)
        native.get().gather_combine(ys, idx, rank, offs, score, k, out)
        ctx.save_for_backward(ys, score, idx, rank, offs)
        ctx.k = k
        return out

    @staticmethod
    def backward(ctx, dout):
        ys, score, idx, rank, offs = ctx.saved_tensors
        dys = torch.empty_like(ys)
        dscore = torch.empty_like(score)
        native.get().combine_bwd(dout.contiguous(), ys, idx, rank, offs, score, ctx.k, dys, dscore)
        return dys, dscore, None, None, None, None


class _ExpertMLP(Function):
    r"""``h4toh(act(htoh4(xs)))`` over expert segments with a fused activation."""

    @staticmethod
    def forward(ctx, xs, w1, b1, w2, b2, offs, act):
        a, pre = gg.forward(xs, w1, offs, b1, act=act, want_pre=True)
        ys = gg.forward(a, w2, offs, b2)
        ctx.save_for_backward(xs, w1, w2, offs, pre, a)
        ctx.act = act
        return ys

    @staticmethod
    def backward(ctx, dys):
        xs, w1, w2, offs, pre, a = ctx.saved_tensors
        groups = w1.shape[0]
        dys = dys.contiguous()
        dw2, db2 = gg.wgrad(dys, a, offs, groups, with_bias_grad=True)
        da = gg.dgrad(dys, w2, offs, pre=pre, act=ctx.act)
        dw1, db1 = gg.wgrad(da, xs, offs, groups, with_bias_grad=True)
        dxs = gg.dgrad(da, w1, offs) if ctx.needs_input_grad[0] else None
        return dxs, dw1, db1, dw2, db2, None, None


class _GroupedLinear(Function):
    r"""One grouped linear over expert segments (used around activations that are not fused)."""

    @staticmethod
    def forward(ctx, xs, w, b, offs):
        ys = gg.forward(xs, w, offs, b)
        ctx.save_for_backward(xs, w, offs)
        return ys

    @staticmethod
    def backward(ctx, dys):
        xs, w, offs = ctx.saved_tensors
        dys = dys.contiguous()
        dw, db = gg.wgrad(dys, xs, offs, w.shape[0], with_bias_grad=True)
        dxs = gg.dgrad(dys, w, offs) if ctx.needs_input_grad[0] else None
        return dxs, dw, db, None


def expert_mlp(layer, xs, offs):
    r"""Both expert linears on rows already grouped by expert (``offs`` on the device)."""
    e = layer.experts
    act = activation_kind(e.activation)
    if act is not None:
        return _ExpertMLP.apply(xs, e.htoh4.weight, e.htoh4.bias, e.h4toh.weight, e.h4toh.bias,
                                offs, act)
    hid = _GroupedLinear.apply(xs, e.htoh4.weight, e.htoh4.bias, offs)
    hid = e.activation(hid)
    return _GroupedLinear.apply(hid.contiguous(), e.h4toh.weight, e.h4toh.bias, offs)


def expert_mlp_weights(xs, offs, w1, b1, w2, b2, activation):
    r"""Both expert linears with explicit weights ``[G, h, d]`` / ``[G, d, h]`` (``activation`` is
    the module between them)."""
    act = activation_kind(activation)
    if act is not None:
        return _ExpertMLP.apply(xs, w1, b1, w2, b2, offs, act)
    hid = _GroupedLinear.apply(xs, w1, b1, offs)
    hid = activation(hid)
    return _GroupedLinear.apply(hid.contiguous(), w2, b2, offs)


def moe_mlp_local(x, gate_idx, gate_score, w1, b1, w2, b2, activation):
    r"""The single-GPU fused MoE MLP over the ``G = w1.shape[0]`` experts given by explicit weights
    (``gate_idx`` in ``[0, G)`` or ``-1`` for slots that take no part).  Used for shadow
    experts, whose parameters arrive by broadcast and are not module parameters."""
    nat = native.get()
    k = gate_idx.shape[1]
    idx = gate_idx.contiguous().view(-1)
    score = gate_score.reshape(-1).to(x.dtype)
    _counts, rank, offs = nat.route_offs(idx, w1.shape[0])
    xs = _Dispatch.apply(x.contiguous(), idx, rank, offs, k)
    ys = expert_mlp_weights(xs, offs, w1.contiguous(), b1.contiguous(), w2.contiguous(), b2.contiguous(),
                            activation)
    return _Combine.apply(ys, score, idx, rank, offs, k)


def moe_mlp_forward(layer, x, gate_idx, gate_score):
    r"""``[B, d] → [B, d]`` for one ``FMoETransformerMLP`` call on the GPU."""
    if layer.world_size > 1 or _forced_ep():
        from ..parallel import symm
        return symm.moe_mlp_forward(layer, x, gate_idx, gate_score)
    nat = native.get()
    k = gate_idx.shape[1]
    idx = gate_idx.contiguous().view(-1)
    score = gate_score.reshape(-1).to(x.dtype)
    with fused_range("route"):
        counts, rank, offs = nat.route_offs(idx, layer.num_expert)
    if config.debug_bounds():
        check_routing(idx, rank, counts, layer.num_expert, offs, idx.numel())
    with fused_range("dispatch"):
        xs = _Dispatch.apply(x.contiguous(), idx, rank, offs, k)
    with fused_range("experts"):
        ys = expert_mlp(layer, xs, offs)
    with fused_range("combine"):
        return _Combine.apply(ys, score, idx, rank, offs, k)
