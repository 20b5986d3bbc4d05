#!/usr/bin/env bash
# Single-node launch:  ./launch/finetune.sh --config configs/qwen3_vl_8b_fsdp_tp2.toml [--training.tp_size 2 ...]
# One process per GPU over NCCL (reference: scripts/finetune.sh:14-18).
set -euo pipefail
NGPUS="${NGPUS:-$(nvidia-smi -L | wc -l)}"
export NCCL_DEBUG="${NCCL_DEBUG:-WARN}"
export PYTHONFAULTHANDLER=1
export OMP_NUM_THREADS="${OMP_NUM_THREADS:-8}"
export WANDB_MODE="${WANDB_MODE:-offline}"
export HF_HUB_OFFLINE="${HF_HUB_OFFLINE:-1}"
python -m vlm_training_b200.ops.build >/dev/null
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node="${NGPUS}" --master-addr 127.0.0.1 \
    --master-port "${MASTER_PORT:-29500}" -m train.train_qwen "$@"
