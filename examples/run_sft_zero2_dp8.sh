#!/bin/bash
# SFT with flat ZeRO sharding over 8 data-parallel ranks, gradients reduced in bf16.
set -euo pipefail
MODEL=${1:?model directory}; DATA=${2:?prompt/answer jsonl}; shift 2
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
  -m cverl_b200.trainer.ppo_trainer --dp 8 --mode sft --sft-jsonl "$DATA" --model-dir "$MODEL" \
  --dp-grad-comm-dtype bfloat16 --master-weights --steps 20 --dtype bfloat16 "$@"
