#!/bin/bash
# enwik8, 12-layer base model (character level).
# Dense feed-forward blocks by default; add "--moe --moe-num-expert 8 --moe-top-k 2" for MoE blocks.
# usage: run_enwik8_base.sh train|eval [N_GPUS] [extra flags]
mode=${1:-train}; gpus=${2:-1}; shift 2 2>/dev/null
launch="python"
[ "$gpus" -gt 1 ] && launch="python -m torch.distributed.run --nnodes=1 --nproc-per-node $gpus --master-addr 127.0.0.1"
common="--data ../data/enwik8 --dataset enwik8 --n_layer 12 --d_model 512 --n_head 8 --d_head 64 --d_inner 2048 --work_dir LM-enwik8-base"
cd "$(dirname "$0")/.."
if [ "$mode" = train ]; then
  $launch train.py $common --dropout 0.1 --dropatt 0.0 --optim adam --lr 0.00025 --warmup_step 0 --max_step 400000 --tgt_len 512 --mem_len 512 --eval_tgt_len 128 --batch_size 22 "$@"
else
  $launch eval.py $common --tgt_len 80 --mem_len 2100 --clamp_len 820 --same_length --split test "$@"
fi
