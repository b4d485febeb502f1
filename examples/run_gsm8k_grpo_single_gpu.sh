#!/bin/bash
# Single-device end-to-end GRPO on a prompt/answer JSONL.
set -euo pipefail
DATA=${1:?prompt/answer jsonl}; MODEL=${2:-}; shift || true; shift || true
if [ -n "$MODEL" ]; then
  exec python -m cverl_b200.trainer.gsm8k_grpo --dataset "$DATA" --policy qwen --model-dir "$MODEL" --tokenizer hf \
    --device cuda:0 --param-dtype bfloat16 --prompts 8 --n 8 --steps 10 --lr 1e-6 "$@"
fi
exec python -m cverl_b200.trainer.gsm8k_grpo --dataset "$DATA" --policy tiny --prompts 8 --n 4 --steps 10 "$@"
