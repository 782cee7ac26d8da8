r"""
The generic MoE layer.

Parity: ``fmoe/layers.py`` — ``FMoE`` (``:87-312``), ``mark_module_parallel_comm``
(``:17-23``) and the private ``_fmoe_general_global_forward`` (``:26-78``).  Behaviour kept:
experts given as ``None`` (caller installs a fused module), a class (instantiated
``num_expert`` times with ``d_model``) or a list of classes; ``slice_group`` with the
deprecated alias ``mp_group``; ``gate_hook(idx, score, None)``; ``mask``/``mask_dict``;
tensor, list or dict inputs; output ``Σ_j score[t,j] · y[t,j]`` with zero rows for dropped
slots.

What differs is the execution: the general path performs one device→host read per call
instead of ``2 + 4·num_expert`` blocking calls, and subclasses with known expert structure
(``FMoETransformerMLP``) bypass it completely on a GPU through ``_fused_forward``.
"""
import torch
import torch.nn as nn

from . import config
from .functions import AllGather, MOEGather, MOEScatter, Slice, ensure_comm, prepare_forward
from .gates import NaiveGate
from .utils import tree


def mark_module_parallel_comm(module, comm):
    r"""Tag every parameter of ``module`` with the name of the group that all-reduces its gradient.

    ``comm`` is one of ``'none'``, ``'dp'``, ``'gate'``, ``'world'`` or a custom group name
    known to :class:`~fastmoe_b200.distributed.DistributedGroupedDataParallel`.
    """
    for p in module.parameters():
        setattr(p, "dp_comm", comm)


def _topk_of(gate_idx):
    return gate_idx.shape[1] if gate_idx.dim() == 2 else 1


def _fmoe_general_global_forward(inp, gate, expert_fn, num_expert, world_size, **kwargs):
    r"""count → scatter → ``expert_fn`` → gather for arbitrary experts and pytree inputs.

    Returns ``[B·top_k, d_out]`` rows in slot order for every output leaf.
    """
    pos, lec, gec, fwd_expert_count, fwd_batch_size = prepare_forward(gate, num_expert, world_size)
    topk = _topk_of(gate)
    token_of_pos = torch.div(pos, topk, rounding_mode="floor")

    x = tree.map_structure(
        lambda t: MOEScatter.apply(t, token_of_pos, lec, gec, fwd_batch_size, world_size), inp)
    x = expert_fn(x, fwd_expert_count)
    out_batch_size = tree.first_leaf(inp).shape[0] * topk
    return tree.map_structure(
        lambda t: MOEGather.apply(t, pos, lec, gec, out_batch_size, world_size), x)


def _general_forward_fn():
    r"""The smart schedule replaces the general forward when ``FMOE_FASTER_SCHEDULE_ENABLE`` is set.

    The reference decides this once at import (``fmoe/layers.py:81-84``); reading the switch
    per call lets tests toggle it.
    """
    if config.faster_schedule_enabled():
        from .fastermoe.schedule import _fmoe_general_global_forward as smart
        return smart, True
    return _fmoe_general_global_forward, False


class FMoE(nn.Module):
    r"""A general MoE layer that accepts arbitrary modules as experts.

    * ``num_expert``: experts on **each** worker.
    * ``world_size``: number of workers holding different experts (expert parallelism).
    * ``slice_group``: group whose members hold identical inputs; each member routes only
      its slice of the batch and the outputs are all-gathered (``mp_group`` is the
      deprecated alias).
    * ``moe_group``: the expert-parallel group (default: all processes).
    * ``top_k``: experts per token.  ``gate``: a gate class from :mod:`fastmoe_b200.gates`.
    * ``expert``: ``None`` | module class | list of module classes.
    * ``gate_bias``: only for ``NaiveGate`` and subclasses.
    """

    def __init__(self, num_expert=32, d_model=1024, world_size=1, mp_group=None,
                 slice_group=None, moe_group=None, top_k=2, gate=NaiveGate, expert=None,
                 gate_hook=None, mask=None, mask_dict=None, gate_bias=True):
        super().__init__()
        self.num_expert = num_expert
        self.d_model = d_model
        self.world_size = world_size

        self.slice_group = slice_group
        if mp_group is not None:
            print("[Warning] mp_group is being deprecated")
            self.slice_group = mp_group
        if self.slice_group is None:
            self.slice_size, self.slice_rank = 1, 0
        else:
            self.slice_size = self.slice_group.size()
            self.slice_rank = self.slice_group.rank()

        self.top_k = top_k
        if isinstance(expert, list):
            self.experts = nn.ModuleList([make(d_model) for make in expert])
            self.experts_fused = False
            self.num_expert = num_expert = len(expert)
        elif expert is not None:
            self.experts = nn.ModuleList([expert(d_model) for _ in range(num_expert)])
            self.experts_fused = False
        else:
            self.experts_fused = True

        if isinstance(gate, type) and issubclass(gate, NaiveGate):
            self.gate = gate(d_model, num_expert, world_size, top_k, gate_bias=gate_bias)
        else:
            self.gate = gate(d_model, num_expert, world_size, top_k)
        self.gate_hook = gate_hook
        self.mask = mask
        self.mask_dict = mask_dict
        self.moe_group = moe_group
        # Gates that exchange counts (capacity limits) must do so inside the layer's own
        # expert-parallel group.  Kept out of the module tree: a group is not a sub-module.
        object.__setattr__(self.gate, "moe_group", moe_group)

    # ------------------------------------------------------------------ expert calls
    def expert_fn(self, inp, fwd_expert_count):
        r"""Run all local experts on rows grouped by expert (``fwd_expert_count`` on the host)."""
        if self.experts_fused:
            return self.experts(inp, fwd_expert_count)
        counts = fwd_expert_count.tolist() if torch.is_tensor(fwd_expert_count) else list(fwd_expert_count)
        outputs, base = [], 0
        for i, n in enumerate(counts):
            n = int(n)
            rows = tree.map_structure(lambda t: t[base:base + n], inp)  # pylint: disable=cell-var-from-loop
            outputs.append(self.experts[i](rows, torch.tensor([n], dtype=torch.int64)))
            base += n
        return tree.map_structure(lambda *parts: torch.cat(parts, dim=0), *outputs)

    def expert_fn_single(self, inp, fwd_expert_count, idx):
        r"""Run local expert ``idx`` alone (used by the smart schedule)."""
        if self.experts_fused:
            if hasattr(self.experts, "forward_single"):
                return self.experts.forward_single(inp, fwd_expert_count, idx)
            raise AssertionError("fused experts without forward_single cannot be scheduled per expert")
        return self.experts[idx](inp, fwd_expert_count)

    def mark_parallel_comm(self, expert_dp_comm="none"):
        r"""Tag expert parameters with ``expert_dp_comm`` and gate parameters with ``'gate'``."""
        experts = getattr(self, "experts", None)
        if experts is not None:
            if isinstance(experts, list):
                for e in experts:
                    mark_module_parallel_comm(e, expert_dp_comm)
            else:
                mark_module_parallel_comm(experts, expert_dp_comm)
        mark_module_parallel_comm(self.gate, "gate")

    # ------------------------------------------------------------------ forward
    def _fused_forward(self, moe_inp, gate_top_k_idx, gate_score):  # pylint: disable=unused-argument
        r"""Hook for subclasses with a fully fused device path; ``None`` = use the general path."""
        return None

    @staticmethod
    def _check_batch(pytree, what):
        rows = {t.shape[0] for t in tree.flatten(pytree)}
        assert len(rows) <= 1, "MoE %s must have the same batch size" % what

    def _route(self, moe_inp):
        r"""Gate call, hook, and the ``[B, k]`` view of the expert ids."""
        ids, scores = self.gate(moe_inp)
        if self.gate_hook is not None:
            self.gate_hook(ids, scores, None)
        if ids.dim() == 1 and self.top_k > 1:
            # Gates that return flattened ids (ZeroGate, NoisyGate in the reference) are
            # given their [B, k] shape back; the reference would treat them as top-1.
            ids = ids.view(-1, self.top_k)
        return ids, scores

    def _unmask(self, rows, mask):
        r"""``[kept * k, d]`` expert outputs → ``[B, k, d]`` with the constant rows of
        ``mask_dict`` at the masked tokens."""
        width = rows.shape[-1]
        full = torch.zeros(mask.shape[0], self.top_k, width, device=rows.device, dtype=rows.dtype)
        full[mask == 0] = rows.view(-1, self.top_k, width)
        for value, constant in self.mask_dict.items():
            full[mask == value] = constant
        return full

    def _general_path(self, moe_inp, ids, scores):
        r"""Arbitrary experts / pytrees / masks: scatter, experts, gather, weighted sum over k."""
        mask = None
        if self.mask is not None and self.mask_dict is not None:
            mask = self.mask.view(-1)
            routed = mask == 0
            moe_inp = tree.map_structure(lambda t: t[routed, :], moe_inp)
            ids = ids[routed, :]

        run, per_expert = _general_forward_fn()
        slots = run(moe_inp, ids, self.expert_fn_single if per_expert else self.expert_fn,
                    self.num_expert, self.world_size, experts=getattr(self, "experts", None))
        if mask is not None:
            per_token = tree.map_structure(lambda t: self._unmask(t, mask), slots)
        else:
            per_token = tree.map_structure(lambda t: t.view(-1, self.top_k, t.shape[-1]), slots)

        weights = scores.view(-1, 1, self.top_k)
        return tree.map_structure(
            lambda t: torch.bmm(weights.to(t.dtype), t).reshape(-1, t.shape[-1]), per_token)

    def forward(self, moe_inp):
        self._check_batch(moe_inp, "inputs")
        if self.world_size > 1:
            tree.map_structure(lambda t: ensure_comm(t, self.moe_group), moe_inp)
        sliced = self.slice_size > 1
        if sliced:
            moe_inp = tree.map_structure(
                lambda t: Slice.apply(t, self.slice_rank, self.slice_size, self.slice_group), moe_inp)

        ids, scores = self._route(moe_inp)
        out = None
        if self.mask is None or self.mask_dict is None:
            out = self._fused_forward(moe_inp, ids, scores)
        if out is None:
            out = self._general_path(moe_inp, ids, scores)

        if sliced:
            out = tree.map_structure(
                lambda t: AllGather.apply(t, self.slice_rank, self.slice_size, self.slice_group), out)
        self._check_batch(out, "outputs")
        return out
