r"""
Wrappers around Megatron's ``forward_step`` / ``loss_func`` / ``model_provider``
(parity: ``fmoe/megatron/patch.py``).

The balance loss of a step is ``mean(layer losses) · balance_loss_weight``, divided by the
pipeline size (each stage only sees its layers) and, from v2.5 on, by the number of
micro-batches; its average over the model-parallel group is reported under
``"<strategy>_loss"``.
"""
import torch


def _unwrap(model):
    while hasattr(model, "module"):
        model = model.module
    return model


def _layer_losses(model, version):
    lm = _unwrap(model).language_model
    if version == "v2.2":
        layers = list(lm.transformer.layers)
    else:
        layers = list(lm.encoder.layers)
        if getattr(lm, "decoder", None) is not None:
            layers += list(lm.decoder.layers)
    return [l.mlp.gate.get_loss(clear=False).view(1) for l in layers if l.mlp.gate.has_loss]


def _average_over_model_parallel(value):
    from megatron.mpu import get_tensor_model_parallel_group
    avg = value.clone().detach()
    if not (torch.distributed.is_available() and torch.distributed.is_initialized()):
        return avg
    group = get_tensor_model_parallel_group()
    torch.distributed.all_reduce(avg, group=group)
    return avg / torch.distributed.get_world_size(group=group)


def patch_loss_func_v2_5(loss_func):
    r"""Megatron ≥ 2.5: ``loss_func(output_tensor)`` → ``loss_func(model, output_tensor)`` with balance loss."""
    from megatron import get_args, get_num_microbatches
    from megatron.mpu import is_pipeline_last_stage
    if not get_args().balance_strategy:
        return loss_func

    def loss_func_with_balance_loss(model, output_tensor):
        args = get_args()
        assert is_pipeline_last_stage(), "Only call loss_func at pipeline last stage."
        loss, state = loss_func(output_tensor)
        losses = _layer_losses(model, "v2.5")
        if not losses:
            return loss, state
        bal = torch.cat(losses).mean() * args.balance_loss_weight / args.pipeline_model_parallel_size
        bal = bal / get_num_microbatches()
        state[args.balance_strategy + "_loss"] = _average_over_model_parallel(bal)
        return loss + bal, state

    return loss_func_with_balance_loss


def patch_forward_step(forward_step_func, Megatron_Version="v2.2"):
    r"""Return a ``forward_step`` that also accounts for the gates' balance losses."""
    from megatron import get_args
    from megatron.mpu import is_pipeline_last_stage
    if not get_args().balance_strategy:
        return forward_step_func

    def forward_step_v2_2(data_iterator, model, input_tensor):
        args = get_args()
        output = forward_step_func(data_iterator, model, input_tensor)
        if not is_pipeline_last_stage() or not args.balance_strategy:
            return output
        losses = _layer_losses(model, "v2.2")
        if not losses:
            return output
        loss, state = output
        bal = torch.cat(losses).mean() * args.balance_loss_weight
        state[args.balance_strategy + "_loss"] = _average_over_model_parallel(bal)
        return loss + bal, state

    def forward_step_v2_5(data_iterator, model):
        from functools import partial
        args = get_args()
        output, loss_func = forward_step_func(data_iterator, model)
        losses = _layer_losses(model, "v2.5")
        bal = torch.cat(losses).mean() * args.balance_loss_weight / args.pipeline_model_parallel_size
        return output, partial(patch_loss_func_v2_5(loss_func), model), bal

    if Megatron_Version == "v2.2":
        return forward_step_v2_2
    if Megatron_Version in ("v2.5", "v3.0.2"):
        return forward_step_v2_5
    raise AssertionError(f"megatron version {Megatron_Version} not known.")


def patch_model_provider(model_provider, gate=None, Megatron_Version="v2.2"):
    r"""Return a ``model_provider`` whose model is already ``fmoefy``-ed.

    The expert hidden size defaults to ``4·hidden / top_k / tensor_parallel_size``, so that the
    compute per token stays that of the dense model.
    """
    from megatron import get_args

    def _hidden_hidden_size(args):
        hhs = args.hidden_size * 4
        assert hhs % args.top_k == 0
        hhs //= args.top_k
        assert hhs % args.tensor_model_parallel_size == 0
        return hhs // args.tensor_model_parallel_size

    def provider_v2_2():
        from .layers import fmoefy
        args = get_args()
        return fmoefy(model_provider(), fmoe_num_experts=args.fmoe_num_experts,
                      hidden_hidden_size=_hidden_hidden_size(args), top_k=args.top_k, gate=gate,
                      megatron_version="v2.2")

    def provider_v2_5(pre_process=True, post_process=True):
        from .layers import fmoefy
        args = get_args()
        return fmoefy(model_provider(pre_process=pre_process, post_process=post_process),
                      fmoe_num_experts=args.fmoe_num_experts,
                      hidden_hidden_size=_hidden_hidden_size(args), top_k=args.top_k, gate=gate,
                      megatron_version=Megatron_Version)

    if Megatron_Version == "v2.2":
        return provider_v2_2
    if Megatron_Version in ("v2.5", "v3.0.2"):
        return provider_v2_5
    raise AssertionError(f"Megatron Version {Megatron_Version} unknown.")
