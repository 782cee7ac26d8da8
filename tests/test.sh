#!/bin/bash
# Run one distributed worker script per rank under SLURM (srun) or OpenMPI (mpirun):
#   srun -N 2 --ntasks-per-node 8 tests/test.sh tests/dist_gpu_worker.py fused_vs_general
# Maps the scheduler's variables to the ones torch.distributed reads and pins one GPU per rank.
if [ -n "$SLURM_PROCID" ]; then
  export RANK=$SLURM_PROCID WORLD_SIZE=$SLURM_NPROCS LOCAL_RANK=$SLURM_LOCALID
  if [ -z "$MASTER_ADDR" ]; then
    export MASTER_ADDR=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)
  fi
elif [ -n "$OMPI_COMM_WORLD_RANK" ]; then
  export RANK=$OMPI_COMM_WORLD_RANK WORLD_SIZE=$OMPI_COMM_WORLD_SIZE
  export LOCAL_RANK=$OMPI_COMM_WORLD_LOCAL_RANK
fi
export MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
export MASTER_PORT=${MASTER_PORT:-29500}
export RANK=${RANK:-0} WORLD_SIZE=${WORLD_SIZE:-1} LOCAL_RANK=${LOCAL_RANK:-0}
exec python "$@"
