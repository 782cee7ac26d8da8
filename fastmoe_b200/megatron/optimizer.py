r"""
Optimizer-side pieces of the Megatron integration.

The reference ships them as source patches to Megatron-LM
(``examples/megatron/clip-grad-v2.2.patch``, ``examples/megatron/v3.0.2.patch:113-207``):

* gradient clipping must count the expert parameters of *all* ranks: their squared norm is
  summed over the group that holds different experts before it joins the dense part;
* the clipping collective runs on every rank in every step — also when an overflow was found or
  clipping is off — because a rank that returns early would leave the others in a collective;
* fp32 master copies inherit the ``dp_comm`` tag of the parameter they shadow.
"""
import torch
import torch.distributed as dist

EXPERT_TAG = "none"


def copy_dp_comm_to_master(param, main_param):
    r"""Give an fp32 master parameter the gradient-reduction tag of its low-precision source."""
    if hasattr(param, "dp_comm"):
        main_param.dp_comm = param.dp_comm
    return main_param


def grad_norm_moe(parameters, norm_type=2, model_parallel_group=None, expert_group=None):
    r"""Global gradient norm of a model whose ``dp_comm == 'none'`` parameters differ per rank.

    ``expert_group`` (default: the world) is the group over which the experts' squared norm is
    summed; ``model_parallel_group`` (optional) the one over which the dense part is summed, as
    in Megatron.  Collective: every rank of the groups must call it.
    """
    assert norm_type == 2, "only the L2 norm is supported with expert parallelism"
    params = [p for p in parameters if p.grad is not None]
    device = params[0].grad.device if params else torch.device("cpu")
    dense = [p.grad.detach().float().pow(2).sum() for p in params
             if getattr(p, "dp_comm", "dp") != EXPERT_TAG]
    expert = [p.grad.detach().float().pow(2).sum() for p in params
              if getattr(p, "dp_comm", "dp") == EXPERT_TAG]
    dense_sq = torch.stack(dense).sum() if dense else torch.zeros((), device=device)
    expert_sq = torch.stack(expert).sum() if expert else torch.zeros((), device=device)
    if dist.is_available() and dist.is_initialized():
        if model_parallel_group is not None:
            dist.all_reduce(dense_sq, group=model_parallel_group)
        # 'cold' ranks without expert gradients still take part
        dist.all_reduce(expert_sq, group=expert_group)
    return (dense_sq + expert_sq).sqrt()


def clip_grad_norm_moe(parameters, max_norm, norm_type=2, model_parallel_group=None,
                       expert_group=None):
    r"""Clip in place to ``max_norm`` (no clipping when ``max_norm <= 0``, but the norm — and its
    collectives — are still computed).  Returns the total norm.  No host read is involved, so
    the call can be captured in a CUDA graph."""
    params = [p for p in parameters if p.grad is not None]
    total = grad_norm_moe(params, norm_type, model_parallel_group, expert_group)
    if max_norm is not None and max_norm > 0 and params:
        coef = (float(max_norm) / (total + 1e-6)).clamp(max=1.0)
        torch._foreach_mul_([p.grad for p in params], coef.to(params[0].grad.dtype))  # pylint: disable=protected-access
    return total
