#!/bin/bash
# WikiText-103, 18-layer large model.
# Dense feed-forward blocks by default; add "--moe --moe-num-expert 8 --moe-top-k 2" for MoE blocks.
# usage: run_wt103_large.sh train|eval [N_GPUS] [extra flags]
mode=${1:-train}; gpus=${2:-1}; shift 2 2>/dev/null
launch="python"
[ "$gpus" -gt 1 ] && launch="python -m torch.distributed.run --nnodes=1 --nproc-per-node $gpus --master-addr 127.0.0.1"
common="--data ../data/wikitext-103 --dataset wt103 --adaptive --div_val 4 --n_layer 18 --d_model 1024 --n_head 16 --d_head 64 --d_inner 4096 --work_dir LM-wt103-large"
cd "$(dirname "$0")/.."
if [ "$mode" = train ]; then
  $launch train.py $common --dropout 0.2 --dropatt 0.2 --optim adam --lr 0.00025 --warmup_step 16000 --max_step 4000000 --tgt_len 384 --mem_len 384 --eval_tgt_len 128 --batch_size 128 "$@"
else
  $launch eval.py $common --tgt_len 128 --mem_len 1600 --clamp_len 1000 --same_length --split test "$@"
fi
