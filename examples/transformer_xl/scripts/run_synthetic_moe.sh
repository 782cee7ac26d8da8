#!/bin/bash
# No dataset needed: Zipf-distributed synthetic tokens; prints ms/batch and tokens/s.
# usage: run_synthetic_moe.sh [N_GPUS] [extra flags]
gpus=${1:-1}; shift 1 2>/dev/null
launch="python"
[ "$gpus" -gt 1 ] && launch="python -m torch.distributed.run --nnodes=1 --nproc-per-node $gpus --master-addr 127.0.0.1"
cd "$(dirname "$0")/.."
$launch train.py --dataset synthetic --n_token 256 --n_layer 12 --d_model 512 --n_head 8 --d_head 64 \
  --d_inner 2048 --tgt_len 512 --mem_len 512 --batch_size 22 --moe --moe-num-expert 8 --moe-top-k 2 \
  --max_step 50 --log-interval 10 --eval-interval 1000000 "$@"
