#!/usr/bin/env bash
# Perplexity of a snapshot on a held-out text file (reference: eval/eval_cat.sh).
#   ./launch/eval_ppl.sh SNAPSHOT val.jsonl
set -euo pipefail
NGPUS="${NGPUS:-1}"
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node="$NGPUS" --master-addr 127.0.0.1 --master-port 29533 \
    -m vlm_training_b200.eval.val --model_dir "$1" --data_path "$2" --seq_len "${SEQ_LEN:-4096}"
