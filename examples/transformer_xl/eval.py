r"""
Evaluate a Transformer-XL checkpoint written by ``train.py`` on one split of a corpus.

Counterpart of the reference's ``examples/transformer-xl/eval.py``: the model is rebuilt from
the same architecture flags, its parameters are loaded from ``--work_dir``, and the attention
lengths can differ from training (``--tgt_len --mem_len --clamp_len --same_length``), which is
how Transformer-XL is evaluated with a longer context than it was trained with.

    python examples/transformer_xl/eval.py --work_dir /tmp/xl --dataset synthetic --split test \
        --n_layer 12 --d_model 512 --n_head 8 --d_head 64 --d_inner 2048 --moe --moe-num-expert 8 \
        --tgt_len 128 --mem_len 1600 --clamp_len 1000 --same_length
"""
import math
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)
from _common import init_distributed, max_over_ranks  # noqa: E402
from data_utils import default_cutoffs, get_lm_corpus  # noqa: E402
import train as xl_train  # noqa: E402

from fastmoe_b200 import checkpoint  # noqa: E402


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    split = "test"
    if "--split" in argv:
        i = argv.index("--split")
        split = argv[i + 1]
        del argv[i:i + 2]
    args = xl_train.get_args(argv)
    assert args.work_dir, "--work_dir with a checkpoint is required"
    rank, world, device = init_distributed()
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dtype]
    if device.type == "cpu":
        dtype = torch.float32
    corpus = get_lm_corpus(args.data, args.dataset, n_token=args.n_token) \
        if args.dataset == "synthetic" else get_lm_corpus(args.data, args.dataset)
    cutoffs = default_cutoffs(args.dataset, corpus.n_token)
    model = xl_train.build_model(args, corpus.n_token, world, cutoffs).to(device).to(dtype)
    step, _ = checkpoint.load(args.work_dir, model)
    iterator = corpus.get_iterator(split, args.batch_size, args.tgt_len, device, args.ext_len, rank, world)
    model.eval()
    total, count, mems = 0.0, 0, ()
    with torch.no_grad():
        for i, (data, target, seq) in enumerate(iterator):
            if 0 < args.max_eval_steps <= i:
                break
            out = model(data, target, *mems)
            total += seq * float(out[0].float().mean())
            count += seq
            mems = out[1:]
    loss = max_over_ranks(total / max(count, 1), device)
    if rank == 0:
        if args.dataset in ("enwik8", "text8"):
            print("| {} loss {:5.3f} | bpc {:7.4f} | checkpoint step {}".format(split, loss, loss / math.log(2), step))
        else:
            print("| {} loss {:5.3f} | ppl {:9.3f} | checkpoint step {}".format(split, loss, math.exp(min(loss, 20.0)), step))
    return loss


if __name__ == "__main__":
    main()
