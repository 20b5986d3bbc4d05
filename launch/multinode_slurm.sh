#!/usr/bin/env bash
#SBATCH --job-name=vlm_b200
#SBATCH --nodes=2
#SBATCH --ntasks-per-node=1
#SBATCH --gpus-per-node=8
#SBATCH --cpus-per-task=64
#SBATCH --exclusive
# Multi-node launch under SLURM: one torchrun agent per node, c10d rendezvous on the first node
# (reference: scripts/multinode_jup.sh:50-58, scripts/multinode_mn5.sh:73-79).
#   sbatch launch/multinode_slurm.sh --config configs/qwen3_vl_8b_fsdp_tp2.toml
set -euo pipefail
HEAD_NODE=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)
HEAD_IP=$(srun --nodes=1 --ntasks=1 -w "$HEAD_NODE" hostname --ip-address | awk '{print $1}')
export NCCL_DEBUG=WARN NCCL_P2P_LEVEL=NVL PYTHONFAULTHANDLER=1 WANDB_MODE=offline HF_HUB_OFFLINE=1
export OMP_NUM_THREADS="${OMP_NUM_THREADS:-8}"
srun ./launch/numa_wrapper.sh python -m torch.distributed.run --nnodes="$SLURM_NNODES" --nproc-per-node=8 \
    --rdzv_id="$SLURM_JOB_ID" --rdzv_backend=c10d --rdzv_endpoint="${HEAD_IP}:29500" -m train.train_qwen "$@"
