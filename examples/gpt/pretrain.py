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

``--pipeline-model-parallel-size P`` splits the layers over ``P`` stages (ranks ``s * world/P ..``
form stage ``s``; experts are spread over the ranks of a stage) and runs ``--num-microbatches``
micro-batches per iteration through the 1F1B runner of :mod:`fastmoe_b200.parallel.pipeline`,
every stage back-propagating ``balance_loss_weight / P`` times the balance loss of its own
gates.  The output embedding of the last stage is not tied to the input embedding of the first.

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
from fastmoe_b200.utils import check_device_status  # noqa: E402
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
    p.add_argument("--pipeline-model-parallel-size", type=int, default=1)
    p.add_argument("--num-microbatches", type=int, default=1)
    add_fmoe_args(p)
    args = p.parse_args()
    if getattr(args, "num_experts", None) is not None:
        args.fmoe_num_experts = args.num_experts
    return args


def main():
    args = get_args()
    rank, world, device = init_distributed()
    pp = args.pipeline_model_parallel_size
    assert world % pp == 0 and args.num_layers % pp == 0
    args.tensor_model_parallel_size = 1
    args.data_parallel_size = world // pp
    args.distributed_experts = args.data_parallel_size > 1
    args.fp16 = args.dtype == "fp16"
    stage, stage_group, prev_rank, next_rank = 0, None, None, None
    if pp > 1:
        from fastmoe_b200.parallel.pipeline import PipelineRunner, build_stage_groups
        stage, stage_group, prev_rank, next_rank = build_stage_groups(pp)
    stub.install(args, data_parallel_group=stage_group, pipeline_rank=stage, pipeline_size=pp,
                 num_microbatches=args.num_microbatches)
    from fastmoe_b200 import megatron as fmoe_megatron

    torch.manual_seed(1234)
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dtype]
    if device.type == "cpu":
        dtype = torch.float32
    cfg = GPTConfig(hidden_size=args.hidden_size, num_layers=args.num_layers,
                    num_attention_heads=args.num_attention_heads, ffn_hidden_size=4 * args.hidden_size,
                    vocab_size=args.vocab_size, max_position_embeddings=args.seq_length,
                    init_method_std=args.init_method_std)

    def model_provider(pre_process=None, post_process=None):
        pre = stage == 0 if pre_process is None else pre_process
        post = stage == pp - 1 if post_process is None else post_process
        return GPTModel(cfg, pre, post, num_layers=args.num_layers // pp)

    if args.fmoefy:
        provider = fmoe_megatron.patch_model_provider(model_provider, Megatron_Version="v3.0.2")
        if args.hidden_hidden_size:
            model = fmoe_megatron.fmoefy(model_provider(), fmoe_num_experts=args.fmoe_num_experts,
                                         distributed_experts=args.distributed_experts,
                                         hidden_hidden_size=args.hidden_hidden_size, top_k=args.top_k,
                                         megatron_version="v3.0.2")
        else:
            model = provider(stage == 0, stage == pp - 1)
        if args.zipf > 0:
            tot = args.fmoe_num_experts * (args.data_parallel_size if args.distributed_experts else 1)
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

    if pp > 1:
        run_pipeline(args, model, ddp, opt, PipelineRunner, stage, pp, prev_rank, next_rank, rank, world,
                     device, dtype, cfg, fmoe_megatron)
        return

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
            check_device_status()   # raises if any kernel reported a peer time-out or an overflow
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


class _Stage(torch.nn.Module):
    r"""A pipeline stage of the GPT: tokens or the previous stage's hidden states in, hidden
    states (logits on the last stage) out."""

    def __init__(self, model):
        super().__init__()
        self.model = model

    def forward(self, x):
        if self.model.pre_process:
            return self.model(x)
        self.model.set_input_tensor(x)
        return self.model(None)


def run_pipeline(args, model, ddp, opt, runner_cls, stage, pp, prev_rank, next_rank, rank, world,
                 device, dtype, cfg, fmoe_megatron):
    stage_size = world // pp
    chain = rank % stage_size

    def lm_loss(logits, labels):
        return torch.nn.functional.cross_entropy(logits.float().reshape(-1, logits.shape[-1]),
                                                 labels.reshape(-1))

    weight = args.balance_loss_weight if (args.fmoefy and args.balance_strategy) else 0.0
    runner = runner_cls(_Stage(model), stage, pp, prev_rank, next_rank,
                        (args.seq_length, args.micro_batch_size, args.hidden_size), dtype,
                        loss_fn=lm_loss, balance_weight=weight, device=device)
    n_micro = args.num_microbatches
    tokens_per_iter = args.micro_batch_size * args.seq_length * stage_size * n_micro
    watch = Stopwatch(device)
    watch.__enter__()
    window = 0
    for it in range(1, args.train_iters + 1):
        # the first and the last stage of a chain draw the same batch
        gen = torch.Generator(device="cpu").manual_seed(4321 + 1000 * it + chain)
        blocks = [torch.randint(0, args.vocab_size, (args.micro_batch_size, args.seq_length + 1), generator=gen)
                  for _ in range(n_micro)]
        tokens = [b[:, :-1].to(device) for b in blocks] if stage == 0 else None
        labels = [b[:, 1:].to(device) for b in blocks] if stage == pp - 1 else None
        opt.zero_grad(set_to_none=True)
        loss = runner.run(micro_batches=tokens, targets=labels, n_micro=n_micro)
        if stage_size > 1:
            ddp.allreduce_params()
        clip_grad_norm_moe(model.parameters(), args.clip_grad)
        opt.step()
        window += 1
        if it % args.log_interval == 0 or it == args.train_iters:
            check_device_status()   # raises if any kernel reported a peer time-out or an overflow
            watch.__exit__()
            ms = max_over_ranks(watch.ms, device) / window
            if rank == world - 1:
                print("iteration {:6d} | ms/iter {:9.2f} | tokens/s {:12.0f} | stages {} x {} | lm loss {:7.4f}".format(
                    it, ms, tokens_per_iter / ms * 1e3, pp, stage_size, float(loss)), flush=True)
            window = 0
            watch.__enter__()
    if args.save:
        fmoe_megatron.save_checkpoint(args.train_iters, ddp, None, None)


if __name__ == "__main__":
    main()
