r"""Topology-aware top-2 gate of FasterMoE (parity: ``fmoe/gates/faster_gate.py:33-116``).

A machine ("node") holds ``FMOE_TOPO_GPUS_PER_NODE`` workers (default 8).  At most
``FMOE_TOPO_OUTGOING_FRACTION`` (default 0.14) of a batch may choose a first expert outside
its own node; everybody else re-picks inside the node.
"""
import torch
import torch.nn.functional as F

from .. import config
from .gshard_gate import gshard_balance_loss
from .naive_gate import NaiveGate


class FasterGate(NaiveGate):
    r"""``FasterGate(d_model, n_expert, world_size, node_rank)``; always top-2."""

    def __init__(self, d_model, n_expert, world_size, node_rank, gate_bias=True):
        super().__init__(d_model, n_expert, world_size, top_k=2, gate_bias=gate_bias)
        self.ne_per_node = config.topo_gpus_per_node() * n_expert
        self.ogn_ratio = config.topo_outgoing_fraction()
        self.node_rank = node_rank
        expert_node = torch.arange(self.tot_expert) // self.ne_per_node
        # True = the expert lives on another node.
        self.register_buffer("mask", expert_node != node_rank, persistent=False)
        self.policy_fn = None

    def forward(self, inp):
        logits = self.gate(inp).view(-1, self.tot_expert)
        remote = self.mask.to(logits.device)
        n_tok = logits.shape[0]

        top2_val, top2_idx = torch.topk(logits, k=2, dim=-1)
        top1_idx = top2_idx[:, 0]
        self.set_loss(gshard_balance_loss(logits, top1_idx, self.tot_expert, self.num_expert))

        with torch.no_grad():
            if self.policy_fn is not None:
                # Experts shadowed on every rank are reachable locally, hence never "remote".
                shadowed = self.policy_fn(top2_idx).view(-1).to(remote.device)
                remote = remote & ~shadowed
            leaves = remote[top1_idx]
            budget = int(n_tok * self.ogn_ratio)
            n_leaving = int(leaves.sum())

        if n_leaving < budget:
            return top2_idx, F.softmax(top2_val, dim=-1)

        with torch.no_grad():
            # The `budget` most confident leaving tokens keep their remote first choice (as
            # second slot); all tokens pick their top-2 among the node-local experts.
            confidence = top2_val[:, 0].detach().clone()
            confidence[~leaves] = float("-inf")
            _, may_leave = torch.topk(confidence, k=budget)
            local_only = logits.detach().clone()
            local_only[:, remote] = float("-inf")
            _, topk_idx = torch.topk(local_only, k=self.top_k)
            topk_idx[may_leave, 1] = top1_idx[may_leave]

        topk_val = torch.gather(logits, 1, topk_idx)
        return topk_idx, F.softmax(topk_val, dim=-1)


def gen_faster_gate(rank):
    r"""Gate factory for worker ``rank`` with the signature ``FMoE`` expects from a gate class."""
    per_node = config.topo_gpus_per_node()

    def _gen(d_model, n_expert, world_size, top_k=2):
        assert top_k == 2
        return FasterGate(d_model, n_expert, world_size, rank // per_node)
    return _gen
