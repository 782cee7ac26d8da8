r"""
Flat views of one expert's parameters and gradients.

Parity: ``fmoe/fastermoe/expert_utils.py:9-72``.  ``e`` is the expert container of an
``FMoE`` layer — a ``ModuleList`` of expert modules or the fused ``_Expert`` — and ``idx``
the local expert index.  Shadowing an expert means shipping these flat buffers: parameters
owner → everybody, gradients everybody → owner.
"""
import torch


def expert_parameters(e, idx):
    r"""The tensors that make up local expert ``idx`` in a fixed order."""
    if isinstance(e, (torch.nn.ModuleList, list, tuple)):
        return [p for _, p in e[idx].named_parameters()]
    if hasattr(e, "htoh4") and hasattr(e, "h4toh"):
        out = []
        for lin in (e.htoh4, e.h4toh):
            out.append(lin.weight[idx])
            if lin.bias is not None:
                out.append(lin.bias[idx])
        return out
    raise TypeError("cannot enumerate the parameters of expert %d in %r" % (idx, type(e)))


def get_expert_param_size(e, idx):
    return sum(p.numel() for p in expert_parameters(e, idx))


def flat_expert_params(e, idx):
    r"""Differentiable 1-D concatenation of the expert's parameters."""
    return torch.cat([p.reshape(-1) for p in expert_parameters(e, idx)])


def get_expert_params(e, out, idx):
    r"""Copy the parameters of expert ``idx`` into the flat buffer ``out``."""
    with torch.no_grad():
        out[:get_expert_param_size(e, idx)].copy_(flat_expert_params(e, idx))


def unflatten_like(e, flat, idx):
    r"""Views of ``flat`` with the shapes of the expert's parameters."""
    views, offset = [], 0
    for p in expert_parameters(e, idx):
        views.append(flat[offset:offset + p.numel()].view(p.shape))
        offset += p.numel()
    return views


def _module_of(e, idx):
    assert isinstance(e, (torch.nn.ModuleList, list, tuple)), "parameter stashing needs per-expert modules"
    return e[idx]


def stash_expert_params(e, params, idx):
    r"""Temporarily replace the parameters of module ``e[idx]`` by ``params`` (flat)."""
    mod = _module_of(e, idx)
    if not hasattr(mod, "expert_param_stash"):
        mod.expert_param_stash, mod.expert_grad_stash = {}, {}
    offset = 0
    for name, p in mod.named_parameters():
        if name not in mod.expert_param_stash:
            mod.expert_param_stash[name] = p.data.clone()
            mod.expert_grad_stash[name] = None if p.grad is None else p.grad.clone()
        with torch.no_grad():
            p.copy_(params[offset:offset + p.numel()].view(p.shape))
        p.grad = None
        offset += p.numel()


def pop_expert_params(e, idx):
    r"""Undo :func:`stash_expert_params`."""
    mod = _module_of(e, idx)
    stash = getattr(mod, "expert_param_stash", None)
    if not stash:
        return
    for name, p in mod.named_parameters():
        with torch.no_grad():
            p.copy_(stash[name])
        if mod.expert_grad_stash[name] is not None:
            p.grad = mod.expert_grad_stash[name].clone()
    mod.expert_param_stash.clear()
    mod.expert_grad_stash.clear()


def collect_expert_grads(e, grads, idx):
    r"""Move the gradients of module ``e[idx]`` into the flat buffer ``grads`` (zeros if absent)."""
    offset = 0
    for _, p in _module_of(e, idx).named_parameters():
        seg = grads[offset:offset + p.numel()]
        if p.grad is None:
            seg.zero_()
        else:
            seg.copy_(p.grad.reshape(-1))
            p.grad = None
        offset += p.numel()


def set_grads(e, grads, idx):
    r"""Accumulate the flat buffer ``grads`` into the gradients of module ``e[idx]``."""
    offset = 0
    for _, p in _module_of(e, idx).named_parameters():
        seg = grads[offset:offset + p.numel()].view(p.shape)
        p.grad = seg.clone() if p.grad is None else p.grad + seg
        offset += p.numel()
