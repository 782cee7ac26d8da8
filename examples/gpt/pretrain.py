r"""
GPT pre-training with ``fmoefy``: every transformer MLP becomes an expert-parallel MoE MLP.

Stand-alone counterpart of the reference's Megatron-LM recipe (``examples/megatron/README.md``
and the ``--fmoefy --num-experts --top-k --balance-strategy`` flags of ``fmoe/megatron/utils.py``):
the model is the Megatron-shaped GPT of :mod:`fastmoe_b200.models.gpt`, the ``megatron`` objects
come from :mod:`fastmoe_b200.megatron.stub` unless Megatron-LM itself is installed, experts are
spread over the data-parallel group (EP = DP = world), gradients go through the grouped DDP and
checkpoints are sharded per data-parallel rank.  ``FMOE_FASTER_SCHEDULE_ENABLE=1`` and
``FMOE_FASTER_SHADOW_ENABLE=1`` turn on the smart schedule and shadow experts.  Tokens are
uniform over the vocabulary (synthetic).

    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 examples/gpt/pretrain.py --fmoefy \
        --num-layers 24 --hidden-size 1024 --num-attention-heads 16 --seq-length 1024 \
        --micro-batch-size 8 --num-experts 2 --top-k 1 --balance-strategy switch --train-iters 20
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from _common import Stopwatch, init_distributed, max_over_ranks  # noqa: E402

from fastmoe_b200.megatron import stub  # noqa: E402
from fastmoe_b200.megatron.optimizer import clip_grad_norm_moe  # noqa: E402
from fastmoe_b200.megatron.utils import add_fmoe_args  # noqa: E402
from fastmoe_b200.models.gpt import GPTConfig, GPTModel, gpt_flops_per_token  # noqa: E402


def get_args():
    p = argparse.ArgumentParser()
    p.add_argument("--num-layers", type=int, default=24)
    p.add_argument("--hidden-size", type=int, default=1024)
    p.add_argument("--num-attention-heads", type=int, default=16)
    p.add_argument("--seq-length", type=int, default=1024)
    p.add_argument("--vocab-size", type=int, default=50257)
    p.add_argument("--micro-batch-size", type=int, default=8)
    p.add_argument("--train-iters", type=int, default=20)
    p.add_argument("--lr", type=float, default=1.5e-4)
    p.add_argument("--init-method-std", type=float, default=0.02)
    p.add_argument("--clip-grad", type=float, default=1.0)
    p.add_argument("--log-interval", type=int, default=5)
    p.add_argument("--save", default=None)
    p.add_argument("--load", default=None)
    p.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"])
    p.add_argument("--zipf", type=float, default=0.0, help="skew of the gate bias (0 = none)")
    add_fmoe_args(p)
    args = p.parse_args()
    if getattr(args, "num_experts", None) is not None:
        args.fmoe_num_experts = args.num_experts
    return args


def main():
    args = get_args()
    rank, world, device = init_distributed()
    args.tensor_model_parallel_size = 1
    args.pipeline_model_parallel_size = 1
    args.data_parallel_size = world
    args.distributed_experts = world > 1
    args.fp16 = args.dtype == "fp16"
    stub.install(args)
    from fastmoe_b200 import megatron as fmoe_megatron

    torch.manual_seed(1234)
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dtype]
    if device.type == "cpu":
        dtype = torch.float32
    cfg = GPTConfig(hidden_size=args.hidden_size, num_layers=args.num_layers,
                    num_attention_heads=args.num_attention_heads, ffn_hidden_size=4 * args.hidden_size,
                    vocab_size=args.vocab_size, max_position_embeddings=args.seq_length,
                    init_method_std=args.init_method_std)

    def model_provider(pre_process=True, post_process=True):
        return GPTModel(cfg, pre_process, post_process)

    if args.fmoefy:
        provider = fmoe_megatron.patch_model_provider(model_provider, Megatron_Version="v3.0.2")
        if args.hidden_hidden_size:
            model = fmoe_megatron.fmoefy(model_provider(), fmoe_num_experts=args.fmoe_num_experts,
                                         distributed_experts=args.distributed_experts,
                                         hidden_hidden_size=args.hidden_hidden_size, top_k=args.top_k,
                                         megatron_version="v3.0.2")
        else:
            model = provider(True, True)
        if args.zipf > 0:
            tot = args.fmoe_num_experts * (world if args.distributed_experts else 1)
            bias = -args.zipf * torch.log(torch.arange(1, tot + 1, dtype=torch.float32))
            for layer in model.language_model.encoder.layers:
                gate = getattr(layer.mlp.gate, "gate", None)
                if gate is not None and gate.bias is not None:
                    with torch.no_grad():
                        gate.bias.copy_(bias)
    else:
        model = model_provider()
    model = model.to(device).to(dtype)
    ddp = fmoe_megatron.DistributedDataParallel(model) if world > 1 else model
    opt = torch.optim.AdamW(model.parameters(), lr=args.lr, weight_decay=0.01)

    gen = torch.Generator(device="cpu").manual_seed(4321 + rank)
    tokens_per_iter = args.micro_batch_size * args.seq_length * world
    watch = Stopwatch(device)
    watch.__enter__()
    window = 0
    for it in range(1, args.train_iters + 1):
        block = torch.randint(0, args.vocab_size, (args.micro_batch_size, args.seq_length + 1), generator=gen)
        tokens, labels = block[:, :-1].to(device), block[:, 1:].to(device)
        lm_loss = ddp(tokens, labels)
        loss = lm_loss
        if args.fmoefy and args.balance_strategy:
            bal = model.balance_losses()
            if bal:
                loss = loss + torch.cat(bal).float().mean() * args.balance_loss_weight
        opt.zero_grad(set_to_none=True)
        loss.backward()
        if world > 1:
            ddp.allreduce_params()
        clip_grad_norm_moe(model.parameters(), args.clip_grad)
        opt.step()
        window += 1
        if it % args.log_interval == 0 or it == args.train_iters:
            watch.__exit__()
            ms = max_over_ranks(watch.ms, device) / window
            if rank == 0:
                hh = args.hidden_hidden_size or (4 * args.hidden_size // max(args.top_k, 1))
                flops = gpt_flops_per_token(cfg, args.top_k if args.fmoefy else 1,
                                            hh if args.fmoefy else None) * tokens_per_iter
                print("iteration {:6d} | ms/iter {:9.2f} | tokens/s {:12.0f} | model TFLOP/s {:8.1f} | lm loss {:7.4f}".format(
                    it, ms, tokens_per_iter / ms * 1e3, flops / ms / 1e9, float(lm_loss)), flush=True)
            window = 0
            watch.__enter__()
    if args.save:
        fmoe_megatron.save_checkpoint(args.train_iters, ddp, None, None)


if __name__ == "__main__":
    main()
