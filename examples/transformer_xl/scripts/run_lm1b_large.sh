#!/bin/bash
# One Billion Word, 24-layer large model.
# Dense feed-forward blocks by default; add "--moe --moe-num-expert 8 --moe-top-k 2" for MoE blocks.
# usage: run_lm1b_large.sh train|eval [N_GPUS] [extra flags]
mode=${1:-train}; gpus=${2:-1}; shift 2 2>/dev/null
launch="python"
[ "$gpus" -gt 1 ] && launch="python -m torch.distributed.run --nnodes=1 --nproc-per-node $gpus --master-addr 127.0.0.1"
common="--data ../data/one-billion-words --dataset lm1b --adaptive --div_val 4 --n_layer 24 --d_model 1280 --n_head 16 --d_head 80 --d_inner 8192 --work_dir LM-lm1b-large"
cd "$(dirname "$0")/.."
if [ "$mode" = train ]; then
  $launch train.py $common --dropout 0.05 --dropatt 0.05 --optim adam --lr 0.00025 --warmup_step 30000 --max_step 1200000 --tgt_len 32 --mem_len 32 --eval_tgt_len 32 --batch_size 512 "$@"
else
  $launch eval.py $common --tgt_len 32 --mem_len 128 --batch_size 8 --split test "$@"
fi
