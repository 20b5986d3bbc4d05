#!/usr/bin/env bash
# Benchmark a converted HF snapshot with lmms-eval on vLLM (reference: scripts/eval.sh).
#   ./launch/eval_benchmarks.sh models/step-1000 [tasks]
set -euo pipefail
MODEL="$1"; TASKS="${2:-docvqa_test,infovqa_test}"
python -m lmms_eval --model vllm --model_args "model=${MODEL},tensor_parallel_size=${TP:-1}" --tasks "$TASKS" \
    --batch_size "${BATCH:-64}" --log_samples --output_path "${OUT:-eval_logs}"
