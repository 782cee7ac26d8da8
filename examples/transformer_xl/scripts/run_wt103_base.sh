#!/bin/bash
# WikiText-103, 16-layer base model (adaptive embedding and softmax).
# Dense feed-forward blocks by default; add "--moe --moe-num-expert 8 --moe-top-k 2" for MoE blocks.
# usage: run_wt103_base.sh train|eval [N_GPUS] [extra flags]
mode=${1:-train}; gpus=${2:-1}; shift 2 2>/dev/null
launch="python"
[ "$gpus" -gt 1 ] && launch="python -m torch.distributed.run --nnodes=1 --nproc-per-node $gpus --master-addr 127.0.0.1"
common="--data ../data/wikitext-103 --dataset wt103 --adaptive --n_layer 16 --d_model 410 --n_head 10 --d_head 41 --d_inner 2100 --work_dir LM-wt103-base"
cd "$(dirname "$0")/.."
if [ "$mode" = train ]; then
  $launch train.py $common --dropout 0.1 --dropatt 0.0 --optim adam --lr 0.00025 --warmup_step 0 --max_step 200000 --tgt_len 150 --mem_len 150 --eval_tgt_len 150 --batch_size 60 "$@"
else
  $launch eval.py $common --tgt_len 64 --mem_len 640 --clamp_len 400 --same_length --split test "$@"
fi
