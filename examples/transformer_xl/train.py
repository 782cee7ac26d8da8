r"""
Transformer-XL language-model training with MoE feed-forward blocks.

Counterpart of the reference's ``examples/transformer-xl/train.py`` (MoE flags ``--moe
--moe-num-expert --moe-top-k`` at ``:144-149`` there; optimisers, schedulers, evaluation
loop, ``--restart`` and ``--multi_gpu`` as in the rest of that file).  Two ways to use
several GPUs:

* one process per GPU (``torchrun``): real expert parallelism — the experts of every MoE block
  are spread over the ranks and ``--moe-num-expert`` counts experts *per GPU*;
* ``--multi_gpu`` in one process: ``torch.nn.DataParallel`` around ``world_size=1`` layers,
  which is what the reference example does.

``--dataset synthetic`` needs no files (a Zipf-distributed token stream); the text corpora are
read from ``--data`` in the layouts of ``data_utils.Corpus``.

    python examples/transformer_xl/train.py --dataset synthetic --n_layer 12 --d_model 512 \
        --n_head 8 --d_head 64 --d_inner 2048 --tgt_len 512 --mem_len 512 --batch_size 22 \
        --moe --moe-num-expert 8 --moe-top-k 2 --max_step 50
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 examples/transformer_xl/train.py ...
"""
import argparse
import math
import os
import sys
import time

import torch
import torch.nn as nn

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)
from _common import Stopwatch, init_distributed, max_over_ranks  # noqa: E402
from data_utils import default_cutoffs, get_lm_corpus  # noqa: E402

from fastmoe_b200 import DistributedGroupedDataParallel, checkpoint  # noqa: E402
from fastmoe_b200.megatron.optimizer import clip_grad_norm_moe  # noqa: E402
from fastmoe_b200.models import MemTransformerLM  # noqa: E402
from fastmoe_b200.utils import check_device_status  # noqa: E402


def get_args(argv=None):
    p = argparse.ArgumentParser(description="Transformer-XL with MoE feed-forward blocks")
    p.add_argument("--data", default=".", help="directory of the corpus files")
    p.add_argument("--dataset", default="synthetic",
                   choices=["synthetic", "wt103", "wt2", "ptb", "enwik8", "text8", "lm1b"])
    p.add_argument("--n_token", type=int, default=256, help="vocabulary size of the synthetic corpus")
    p.add_argument("--n_layer", type=int, default=12)
    p.add_argument("--n_head", type=int, default=8)
    p.add_argument("--d_head", type=int, default=64)
    p.add_argument("--d_embed", type=int, default=-1)
    p.add_argument("--d_model", type=int, default=512)
    p.add_argument("--d_inner", type=int, default=2048)
    p.add_argument("--dropout", type=float, default=0.1)
    p.add_argument("--dropatt", type=float, default=0.0)
    p.add_argument("--optim", default="adam", choices=["adam", "sgd", "adagrad"])
    p.add_argument("--lr", type=float, default=2.5e-4)
    p.add_argument("--mom", type=float, default=0.0)
    p.add_argument("--scheduler", default="cosine", choices=["cosine", "inv_sqrt", "dev_perf", "constant"])
    p.add_argument("--warmup_step", type=int, default=0)
    p.add_argument("--decay_rate", type=float, default=0.5)
    p.add_argument("--lr_min", type=float, default=0.0)
    p.add_argument("--eta_min", type=float, default=0.0)
    p.add_argument("--patience", type=int, default=0)
    p.add_argument("--clip", type=float, default=0.25)
    p.add_argument("--max_step", type=int, default=100)
    p.add_argument("--batch_size", type=int, default=22, help="sequences per process")
    p.add_argument("--batch_chunk", type=int, default=1, help="split a batch to save memory")
    p.add_argument("--tgt_len", type=int, default=512)
    p.add_argument("--eval_tgt_len", type=int, default=128)
    p.add_argument("--ext_len", type=int, default=0)
    p.add_argument("--mem_len", type=int, default=512)
    p.add_argument("--not_tied", action="store_true")
    p.add_argument("--seed", type=int, default=1111)
    p.add_argument("--adaptive", action="store_true", help="adaptive embedding and softmax")
    p.add_argument("--div_val", type=int, default=1)
    p.add_argument("--pre_lnorm", action="store_true")
    p.add_argument("--varlen", action="store_true")
    p.add_argument("--multi_gpu", action="store_true", help="nn.DataParallel in one process")
    p.add_argument("--gpu0_bsz", type=int, default=-1,
                   help="with --multi_gpu: sequences of a batch given to GPU 0 (it also gathers)")
    p.add_argument("--sample_softmax", type=int, default=-1,
                   help="train against this many log-uniform negatives instead of the full softmax")
    p.add_argument("--same_length", action="store_true")
    p.add_argument("--clamp_len", type=int, default=-1)
    p.add_argument("--log-interval", type=int, default=10)
    p.add_argument("--eval-interval", type=int, default=4000)
    p.add_argument("--max_eval_steps", type=int, default=-1)
    p.add_argument("--work_dir", default=None)
    p.add_argument("--restart", action="store_true")
    p.add_argument("--restart_dir", default="")
    p.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"])
    p.add_argument("--moe", action="store_true")
    p.add_argument("--moe-num-expert", type=int, default=8, help="experts per GPU")
    p.add_argument("--moe-top-k", type=int, default=2)
    p.add_argument("--balance-weight", type=float, default=0.0)
    args = p.parse_args(argv)
    assert args.batch_size % args.batch_chunk == 0
    return args


def build_model(args, n_token, world, cutoffs):
    return MemTransformerLM(
        n_token, args.n_layer, args.n_head, args.d_model, args.d_head, args.d_inner, args.dropout,
        args.dropatt, tie_weight=not args.not_tied, pre_lnorm=args.pre_lnorm, tgt_len=args.tgt_len,
        ext_len=args.ext_len, mem_len=args.mem_len, same_length=args.same_length,
        clamp_len=args.clamp_len, moe=args.moe, moe_num_expert=args.moe_num_expert,
        moe_top_k=args.moe_top_k, world_size=world if args.moe else 1,
        d_embed=args.d_embed, cutoffs=cutoffs if args.adaptive else (), div_val=args.div_val,
        tie_projs=[False] + [True] * len(cutoffs) if args.adaptive else (),
        sample_softmax=args.sample_softmax)


def build_optimizer(args, model):
    if args.optim == "sgd":
        return torch.optim.SGD(model.parameters(), lr=args.lr, momentum=args.mom)
    if args.optim == "adagrad":
        return torch.optim.Adagrad(model.parameters(), lr=args.lr)
    return torch.optim.Adam(model.parameters(), lr=args.lr)


def build_scheduler(args, opt):
    if args.scheduler == "cosine":
        return torch.optim.lr_scheduler.CosineAnnealingLR(opt, args.max_step, eta_min=args.eta_min)
    if args.scheduler == "inv_sqrt":
        def factor(step):
            if step == 0 and args.warmup_step == 0:
                return 1.0
            if step > args.warmup_step:
                return 1.0 / math.sqrt(step)
            return step / (args.warmup_step ** 1.5)
        return torch.optim.lr_scheduler.LambdaLR(opt, lr_lambda=factor)
    if args.scheduler == "dev_perf":
        return torch.optim.lr_scheduler.ReduceLROnPlateau(opt, factor=args.decay_rate,
                                                          patience=args.patience, min_lr=args.lr_min)
    return None


def evaluate(args, model, iterator, device, max_steps=-1):
    r"""Mean loss over an evaluation split with the evaluation lengths (longer memory)."""
    model.eval()
    model.reset_length(args.eval_tgt_len, args.ext_len,
                       args.mem_len + args.tgt_len - args.eval_tgt_len if args.mem_len > 0 else 0)
    total, count, mems = 0.0, 0, ()
    with torch.no_grad():
        for i, (data, target, seq) in enumerate(iterator):
            if 0 < max_steps <= i:
                break
            out = model(data, target, *mems)
            loss, mems = out[0], out[1:]
            total += seq * float(loss.float().mean())
            count += seq
    model.reset_length(args.tgt_len, args.ext_len, args.mem_len)
    model.train()
    return total / max(count, 1)


def main(argv=None):
    args = get_args(argv)
    rank, world, device = init_distributed()
    torch.manual_seed(args.seed)
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dtype]
    if device.type == "cpu":
        dtype = torch.float32

    corpus = get_lm_corpus(args.data, args.dataset, n_token=args.n_token) \
        if args.dataset == "synthetic" else get_lm_corpus(args.data, args.dataset)
    n_token = corpus.n_token
    cutoffs = default_cutoffs(args.dataset, n_token)
    tr_iter = corpus.get_iterator("train", args.batch_size, args.tgt_len, device, args.ext_len, rank, world)
    va_iter = corpus.get_iterator("valid", max(1, args.batch_size // 2), args.eval_tgt_len, device,
                                  args.ext_len, rank, world)

    model = build_model(args, n_token, world, cutoffs).to(device).to(dtype)
    if args.multi_gpu and world == 1 and torch.cuda.device_count() > 1:
        if args.gpu0_bsz >= 0:
            from exp_utils import BalancedDataParallel
            para_model = BalancedDataParallel(args.gpu0_bsz // args.batch_chunk, model, dim=1)
        else:
            para_model = nn.DataParallel(model, dim=1)   # batch is dimension 1 of [seq, batch]
    elif world > 1:
        para_model = DistributedGroupedDataParallel(model)
    else:
        para_model = model
    opt = build_optimizer(args, model)
    sched = build_scheduler(args, opt)
    step, best_val = 0, None
    restart_dir = args.restart_dir or args.work_dir
    if args.restart and restart_dir:
        loaded, _ = checkpoint.load(restart_dir, model, opt)
        step = loaded or 0
    log = print
    if rank == 0 and args.work_dir:
        from exp_utils import create_exp_dir
        log = create_exp_dir(args.work_dir, scripts_to_save=[os.path.abspath(__file__)])
    if rank == 0:
        n_all = sum(p.numel() for p in model.parameters())
        n_exp = sum(p.numel() for p in model.parameters() if getattr(p, "dp_comm", "dp") == "none")
        log("| params/rank {:,} (experts {:,}) | vocab {} | ranks {}".format(n_all, n_exp, n_token, world))

    tokens_per_step = args.tgt_len * args.batch_size * world
    model.train()
    watch = Stopwatch(device).__enter__()
    window, window_loss = 0, 0.0
    mems = [()] * args.batch_chunk
    t_start = time.time()
    while step < args.max_step:
        it = tr_iter.get_varlen_iter() if args.varlen else tr_iter.get_fixlen_iter()
        for data, target, _seq in it:
            opt.zero_grad(set_to_none=True)
            data_chunks = torch.chunk(data, args.batch_chunk, dim=1)
            target_chunks = torch.chunk(target, args.batch_chunk, dim=1)
            loss_value = 0.0
            for c, (d_c, t_c) in enumerate(zip(data_chunks, target_chunks)):
                out = para_model(d_c.contiguous(), t_c.contiguous(), *mems[c])
                loss, mems[c] = out[0].float().mean() / args.batch_chunk, out[1:]
                total = loss
                if args.moe and args.balance_weight > 0:
                    bal = model.balance_losses()
                    if bal:
                        total = total + args.balance_weight * torch.cat(bal).float().mean() / args.batch_chunk
                total.backward()
                loss_value += float(loss.detach())
            if world > 1:
                para_model.allreduce_params()
            clip_grad_norm_moe(model.parameters(), args.clip)
            opt.step()
            step += 1
            if args.scheduler in ("cosine", "constant", "dev_perf") and step < args.warmup_step:
                for group in opt.param_groups:
                    group["lr"] = args.lr * step / args.warmup_step
            elif sched is not None and args.scheduler != "dev_perf":
                sched.step()
            window += 1
            window_loss += loss_value
            if step % args.log_interval == 0 or step == args.max_step:
                check_device_status()   # raises if any kernel reported a peer time-out or an overflow
                watch.__exit__()
                ms = max_over_ranks(watch.ms, device) / window
                if rank == 0:
                    mean = window_loss / window
                    unit = "bpc {:6.4f}".format(mean / math.log(2)) if args.dataset in ("enwik8", "text8") \
                        else "ppl {:9.3f}".format(math.exp(min(mean, 20.0)))
                    log("| step {:6d} | lr {:.3g} | ms/batch {:8.2f} | tokens/s {:12.0f} | loss {:5.3f} | {}".format(
                        step, opt.param_groups[0]["lr"], ms, tokens_per_step / ms * 1e3, mean, unit))
                window, window_loss = 0, 0.0
                watch.__enter__()
            if step % args.eval_interval == 0 or step == args.max_step:
                val = evaluate(args, model, va_iter.get_fixlen_iter(), device, args.max_eval_steps)
                val = max_over_ranks(val, device) if world > 1 else val
                if rank == 0:
                    log("| eval at step {:6d} | {:6.1f} s | valid loss {:5.3f}".format(
                        step, time.time() - t_start, val))
                if args.work_dir and (best_val is None or val < best_val):
                    checkpoint.save(args.work_dir, step, model, opt)
                    best_val = val
                if args.scheduler == "dev_perf" and sched is not None:
                    sched.step(val)
                watch.__enter__()
            if step >= args.max_step:
                break
    if args.work_dir and best_val is None:
        checkpoint.save(args.work_dir, step, model, opt)


if __name__ == "__main__":
    main()
