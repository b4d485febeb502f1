#!/bin/bash
# Context parallel CP=8: one long sequence sharded over 8 GPUs (ring attention, conv halo, state hand-off).
set -euo pipefail
MODEL=${1:-}; shift || true
ARGS=(--cp 8 --prompt-len 1024 --response-len 31744 --steps 3 --dtype bfloat16)
if [ -n "$MODEL" ]; then ARGS+=(--model-dir "$MODEL"); else ARGS+=(--config qwen3_5_0_8b --max-layers 4); fi
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
  -m cverl_b200.trainer.ppo_trainer "${ARGS[@]}" "$@"
