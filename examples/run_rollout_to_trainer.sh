#!/bin/bash
# Rollout files -> distributed trainer: first an engine (a vLLM server over HTTP, or the built-in oracle) writes
# rollout_step_%06d.json into ROLLOUT_DIR without training, then the distributed trainer consumes the directory
# step by step (the flow of the reference's tools/distributed/run_rollout_to_pp_tp_ppo.sh).
#   DATASET=gsm8k.jsonl examples/run_rollout_to_trainer.sh MODEL_DIR [extra trainer flags]
# ROLLOUT_BACKEND=http VLLM_BASE_URL=http://127.0.0.1:8000 SERVED_MODEL_NAME=... use a running server.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
MODEL_DIR=${1:?model directory (config.json + safetensors; tokenizer.json for a BPE vocabulary)}; shift
DATASET=${DATASET:?DATASET=<prompt/answer jsonl>}
export ROLLOUT_DIR=${ROLLOUT_DIR:-${TMPDIR:-/tmp}/cverl_b200_rollouts}
export PP_SIZE=${PP_SIZE:-2} TP_SIZE=${TP_SIZE:-2} MICRO_BATCHES=${MICRO_BATCHES:-4} PROMPT_LEN=${PROMPT_LEN:-128}
export RESPONSE_LEN=${RESPONSE_LEN:-64} STEPS=${STEPS:-5} LR=${LR:-1e-10} LAYERS=${LAYERS:--1}
PROMPTS=${PROMPTS:-2}; N=${N:-2}
mkdir -p "$ROLLOUT_DIR"
find "$ROLLOUT_DIR" -maxdepth 1 -name 'rollout_step_*.json' -delete
python -m cverl_b200.cli.online_grpo --model-dir "$MODEL_DIR" --dataset "$DATASET" \
  --rollout "${ROLLOUT_BACKEND:-oracle}" --server "${VLLM_BASE_URL:-http://127.0.0.1:8000}" \
  --served-model "${SERVED_MODEL_NAME:-$MODEL_DIR}" --skip-train --dump-rollout-dir "$ROLLOUT_DIR" \
  --steps "$STEPS" --prompts "$PROMPTS" --n "$N" --max-prompt-tokens "$PROMPT_LEN" --max-response-tokens "$RESPONSE_LEN" \
  --max-layers "$LAYERS"
[ -f "$MODEL_DIR/tokenizer.json" ] && export TOKENIZER_JSON=${TOKENIZER_JSON:-$MODEL_DIR/tokenizer.json}
exec "$HERE/run_pp_tp_ppo_trainer.sh" "$MODEL_DIR" "$@"
