r"""
Plug-ins for Megatron-LM (parity: ``fmoe/megatron/__init__.py:4-20``).

``fmoefy`` swaps the MLP of every transformer layer for an expert-parallel MoE MLP,
``patch_forward_step`` / ``patch_model_provider`` wire the balance loss and the swap into
Megatron's training loop, ``DistributedDataParallel`` replaces Megatron's local DDP,
``save_checkpoint`` / ``load_checkpoint`` shard expert parameters per data-parallel rank.
Everything reads Megatron through ``import megatron`` at call time; where Megatron-LM is not
installed, :mod:`fastmoe_b200.megatron.stub` provides the few objects that are needed
(``get_args``, ``mpu``, ``checkpointing``) so that the adapter and the GPT example run
stand-alone.
"""
from .utils import add_fmoe_args
from .layers import MegatronMLP, fmoefy
from .checkpoint import load_checkpoint, save_checkpoint
from .distributed import DistributedDataParallel
from .balance import (add_balance_log, generate_megatron_gate_hook, get_balance_profile,
                      reset_gate_hook)
from .patch import patch_forward_step, patch_model_provider
from .optimizer import clip_grad_norm_moe, copy_dp_comm_to_master, grad_norm_moe

__all__ = ["add_fmoe_args", "MegatronMLP", "fmoefy", "save_checkpoint", "load_checkpoint",
           "DistributedDataParallel", "reset_gate_hook", "get_balance_profile",
           "generate_megatron_gate_hook", "add_balance_log", "patch_forward_step",
           "patch_model_provider", "clip_grad_norm_moe", "grad_norm_moe", "copy_dp_comm_to_master"]
