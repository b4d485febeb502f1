#!/bin/bash
# Qwen3-MoE SFT on PP=2 x TP=2 x EP=2.
set -euo pipefail
MODEL=${1:-}; shift || true
ARGS=(--pp 2 --tp 2 --ep 2 --micro-batches 4 --steps 5 --dtype bfloat16)
if [ -n "$MODEL" ]; then ARGS+=(--model-dir "$MODEL"); else ARGS+=(--config tiny_moe); fi
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
  -m cverl_b200.trainer.ppo_trainer "${ARGS[@]}" "$@"
