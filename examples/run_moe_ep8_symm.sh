#!/bin/bash
# Qwen3-MoE SFT with expert parallelism EP=8, token dispatch / combine by row scatter / gather kernels over
# NVLink peer memory.  Without a model directory: the Qwen3-30B-A3B shape, random weights, 16 of its 48 layers.
set -euo pipefail
MODEL=${1:-}; shift || true
ARGS=(--ep 8 --ep-comm symm --mode sft --prompt-len 256 --response-len 1024 --micro-batch-seqs 4 --steps 4 --dtype bfloat16)
if [ -n "$MODEL" ]; then ARGS+=(--model-dir "$MODEL"); else ARGS+=(--config qwen3_30b_a3b --max-layers 16 --rows 16); fi
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
  -m cverl_b200.trainer.ppo_trainer "${ARGS[@]}" "$@"
