#!/bin/bash
# GRPO actor update on 8 GPUs: DP=4 x TP=2 (the headline configuration).
set -euo pipefail
MODEL=${1:-}; shift || true
ARGS=(--dp 4 --tp 2 --mode ppo --micro-batches 8 --micro-batch-seqs 16 --prompt-len 256 --response-len 1024
      --steps 10 --dtype bfloat16 --zero-comm symm --max-grad-norm 1.0 --metrics-csv grpo_dp4_tp2.csv)
if [ -n "$MODEL" ]; then ARGS+=(--model-dir "$MODEL"); else ARGS+=(--config qwen3_5_0_8b); fi
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
  -m cverl_b200.trainer.ppo_trainer "${ARGS[@]}" "$@"
