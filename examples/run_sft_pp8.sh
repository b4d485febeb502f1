#!/bin/bash
# SFT with an 8-stage pipeline (1F1B, 16 micro-batches).
set -euo pipefail
MODEL=${1:?model directory}; DATA=${2:?prompt/answer jsonl}; shift 2
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
  -m cverl_b200.trainer.ppo_trainer --pp 8 --mode sft --sft-jsonl "$DATA" --model-dir "$MODEL" \
  --micro-batches 16 --steps 20 --dtype bfloat16 --checkpoint-dir ckpt_sft_pp8 --checkpoint-every 10 "$@"
