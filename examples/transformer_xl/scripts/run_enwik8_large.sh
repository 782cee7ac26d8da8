#!/bin/bash
# enwik8, 24-layer large model.
# Dense feed-forward blocks by default; add "--moe --moe-num-expert 8 --moe-top-k 2" for MoE blocks.
# usage: run_enwik8_large.sh train|eval [N_GPUS] [extra flags]
mode=${1:-train}; gpus=${2:-1}; shift 2 2>/dev/null
launch="python"
[ "$gpus" -gt 1 ] && launch="python -m torch.distributed.run --nnodes=1 --nproc-per-node $gpus --master-addr 127.0.0.1"
common="--data ../data/enwik8 --dataset enwik8 --n_layer 24 --d_model 1024 --n_head 8 --d_head 128 --d_inner 3072 --work_dir LM-enwik8-large"
cd "$(dirname "$0")/.."
if [ "$mode" = train ]; then
  $launch train.py $common --dropout 0.15 --dropatt 0.15 --optim adam --lr 0.00025 --warmup_step 4000 --max_step 400000 --tgt_len 768 --mem_len 768 --eval_tgt_len 128 --batch_size 64 "$@"
else
  $launch eval.py $common --tgt_len 128 --mem_len 3800 --clamp_len 1000 --same_length --split test "$@"
fi
