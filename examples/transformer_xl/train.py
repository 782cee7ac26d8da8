r"""
Transformer-XL language-model training with expert-parallel MoE feed-forward blocks.

Counterpart of the reference's ``examples/transformer-xl/train.py`` (flags ``--moe
--moe-num-expert --moe-top-k`` at ``:144-149`` there), but one process per GPU with real expert
parallelism instead of ``nn.DataParallel`` around ``world_size=1`` layers.  ``--data synthetic``
draws tokens uniformly from the vocabulary (no dataset is needed); a text file can be given
instead and is read as bytes.

    python examples/transformer_xl/train.py --n_layer 12 --d_model 512 --n_head 8 --d_head 64 \
        --d_inner 2048 --tgt_len 512 --mem_len 512 --batch_size 22 --moe --moe-num-expert 8 \
        --moe-top-k 2 --max_step 50
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 examples/transformer_xl/train.py ...
"""
import argparse
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from _common import Stopwatch, init_distributed, max_over_ranks  # noqa: E402

from fastmoe_b200 import DistributedGroupedDataParallel, checkpoint  # noqa: E402
from fastmoe_b200.megatron.optimizer import clip_grad_norm_moe  # noqa: E402
from fastmoe_b200.models import MemTransformerLM  # noqa: E402


def get_args():
    p = argparse.ArgumentParser()
    p.add_argument("--data", default="synthetic")
    p.add_argument("--n_token", type=int, default=256)
    p.add_argument("--n_layer", type=int, default=12)
    p.add_argument("--n_head", type=int, default=8)
    p.add_argument("--d_head", type=int, default=64)
    p.add_argument("--d_model", type=int, default=512)
    p.add_argument("--d_inner", type=int, default=2048)
    p.add_argument("--dropout", type=float, default=0.1)
    p.add_argument("--dropatt", type=float, default=0.0)
    p.add_argument("--lr", type=float, default=2.5e-4)
    p.add_argument("--clip", type=float, default=0.25)
    p.add_argument("--max_step", type=int, default=100)
    p.add_argument("--warmup_step", type=int, default=0)
    p.add_argument("--batch_size", type=int, default=22, help="sequences per GPU")
    p.add_argument("--tgt_len", type=int, default=512)
    p.add_argument("--mem_len", type=int, default=512)
    p.add_argument("--ext_len", type=int, default=0)
    p.add_argument("--pre_lnorm", action="store_true")
    p.add_argument("--not_tied", action="store_true")
    p.add_argument("--seed", type=int, default=1111)
    p.add_argument("--log-interval", type=int, default=10)
    p.add_argument("--work_dir", default=None)
    p.add_argument("--restart", action="store_true")
    p.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"])
    p.add_argument("--moe", action="store_true")
    p.add_argument("--moe-num-expert", type=int, default=8, help="experts per GPU")
    p.add_argument("--moe-top-k", type=int, default=2)
    p.add_argument("--balance-weight", type=float, default=0.0)
    return p.parse_args()


def batches(args, device, rank):
    gen = torch.Generator(device="cpu").manual_seed(args.seed + rank)
    if args.data == "synthetic":
        while True:
            block = torch.randint(0, args.n_token, (args.tgt_len + 1, args.batch_size), generator=gen)
            yield block[:-1].to(device), block[1:].to(device)
    else:
        raw = torch.tensor(list(open(args.data, "rb").read()), dtype=torch.long)
        n = raw.numel() // args.batch_size
        stream = raw[:n * args.batch_size].view(args.batch_size, n).t().contiguous()
        pos = 0
        while True:
            if pos + args.tgt_len + 1 > n:
                pos = 0
            yield (stream[pos:pos + args.tgt_len].to(device),
                   stream[pos + 1:pos + 1 + args.tgt_len].to(device))
            pos += args.tgt_len


def main():
    args = get_args()
    rank, world, device = init_distributed()
    torch.manual_seed(args.seed)
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dtype]
    if device.type == "cpu":
        dtype = torch.float32
    model = MemTransformerLM(args.n_token, args.n_layer, args.n_head, args.d_model, args.d_head,
                             args.d_inner, args.dropout, args.dropatt, tie_weight=not args.not_tied,
                             pre_lnorm=args.pre_lnorm, tgt_len=args.tgt_len, ext_len=args.ext_len,
                             mem_len=args.mem_len, moe=args.moe, moe_num_expert=args.moe_num_expert,
                             moe_top_k=args.moe_top_k, world_size=world if args.moe else 1)
    model = model.to(device).to(dtype)
    para_model = DistributedGroupedDataParallel(model) if world > 1 else model
    opt = torch.optim.Adam(model.parameters(), lr=args.lr)
    sched = torch.optim.lr_scheduler.CosineAnnealingLR(opt, args.max_step)
    step = 0
    if args.restart and args.work_dir:
        loaded, _ = checkpoint.load(args.work_dir, model, opt)
        step = loaded or 0

    data = batches(args, device, rank)
    mems = ()
    tokens_per_step = args.tgt_len * args.batch_size * world
    model.train()
    watch = Stopwatch(device)
    watch.__enter__()
    window = 0
    while step < args.max_step:
        inp, tgt = next(data)
        out = para_model(inp, tgt, *mems)
        loss, mems = out[0].float().mean(), out[1:]
        total = loss
        if args.moe and args.balance_weight > 0:
            bal = model.balance_losses()
            if bal:
                total = total + args.balance_weight * torch.cat(bal).float().mean()
        opt.zero_grad(set_to_none=True)
        total.backward()
        if world > 1:
            para_model.allreduce_params()
        clip_grad_norm_moe(model.parameters(), args.clip)
        opt.step()
        sched.step()
        step += 1
        window += 1
        if step % args.log_interval == 0 or step == args.max_step:
            watch.__exit__()
            ms = max_over_ranks(watch.ms, device) / window
            if rank == 0:
                print("| step {:6d} | lr {:.3g} | ms/batch {:8.2f} | tokens/s {:12.0f} | loss {:5.3f} | bpc {:6.4f}".format(
                    step, sched.get_last_lr()[0], ms, tokens_per_step / ms * 1e3, float(loss),
                    float(loss) / math.log(2)), flush=True)
            window = 0
            watch.__enter__()
    if args.work_dir:
        checkpoint.save(args.work_dir, step, model, opt)


if __name__ == "__main__":
    main()
