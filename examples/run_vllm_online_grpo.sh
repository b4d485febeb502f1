#!/bin/bash
# Online GRPO against a vLLM server with the weights pushed back over NCCL after every update: starts `vllm serve`
# on VLLM_GPUS (tensor parallel VLLM_TP_SIZE, sleep mode and the NCCL weight-transfer engine enabled), waits for it,
# asks it for its world size and runs the loop on TRAINER_GPUS.  One script for the reference's three launchers
# (examples/run_vllm_online_grpo.sh, run_vllm_tp2_online_grpo_h20.sh, run_vllm_static_split_4gpu_h20.sh):
#   MODEL_DIR=... DATASET=gsm8k.jsonl examples/run_vllm_online_grpo.sh                       # 1 + 1 GPUs
#   VLLM_GPUS=0,1 VLLM_TP_SIZE=2 TRAINER_GPUS=2 ... examples/run_vllm_online_grpo.sh         # tp 2 server
#   STATIC_SPLIT=1 ... : the server only generates (rollout files under ROLLOUT_DIR, no update, no weight push)
# DRY_RUN=1 prints the two command lines and exits; ROLLOUT_BACKEND=oracle needs no server at all.
set -euo pipefail
MODEL_DIR=${MODEL_DIR:?MODEL_DIR=<model directory>}
DATASET=${DATASET:?DATASET=<prompt/answer jsonl>}
HOST=${HOST:-127.0.0.1}; PORT=${PORT:-8001}
BASE_URL=${VLLM_BASE_URL:-http://$HOST:$PORT}
SERVED_MODEL_NAME=${SERVED_MODEL_NAME:-cverl-policy}
VLLM_GPUS=${VLLM_GPUS:-0}; TRAINER_GPUS=${TRAINER_GPUS:-1}
VLLM_LOG=${VLLM_LOG:-${TMPDIR:-/tmp}/cverl_b200_vllm.log}
BACKEND=${ROLLOUT_BACKEND:-http}
SERVE=(vllm serve "$MODEL_DIR" --served-model-name "$SERVED_MODEL_NAME" --host "$HOST" --port "$PORT"
       --dtype "${VLLM_DTYPE:-bfloat16}" --tensor-parallel-size "${VLLM_TP_SIZE:-1}"
       --gpu-memory-utilization "${VLLM_GPU_MEMORY_UTILIZATION:-0.70}" --enable-sleep-mode
       --weight-transfer-config '{"backend":"nccl"}')
LOOP=(python -m cverl_b200.cli.online_grpo --model-dir "$MODEL_DIR" --dataset "$DATASET" --rollout "$BACKEND"
      --server "$BASE_URL" --served-model "$SERVED_MODEL_NAME" --device "${DEVICE:-cuda:0}"
      --param-dtype "${PARAM_DTYPE:-bfloat16}" --max-layers "${MAX_LAYERS:--1}" --steps "${STEPS:-1}"
      --prompts "${PROMPTS:-1}" --n "${N:-2}" --max-prompt-tokens "${MAX_PROMPT_TOKENS:-64}"
      --max-response-tokens "${MAX_RESPONSE_TOKENS:-64}" --ppo-epochs "${PPO_EPOCHS:-1}" --lr "${LR:-3e-6}")
[ -n "${ROLLOUT_DIR:-}" ] && LOOP+=(--dump-rollout-dir "$ROLLOUT_DIR")
if [ "${STATIC_SPLIT:-0}" = "1" ]; then
  LOOP+=(--skip-train)
elif [ "$BACKEND" = "http" ]; then
  LOOP+=(--weight-sync nccl --weight-master-address "${MASTER_ADDRESS:-127.0.0.1}" --weight-master-port "${MASTER_PORT:-29601}")
  [ "${SLEEP_DURING_TRAIN:-0}" = "1" ] && LOOP+=(--sleep-during-train)
fi
if [ "${DRY_RUN:-0}" = "1" ]; then
  [ "$BACKEND" = "http" ] && echo "CUDA_VISIBLE_DEVICES=$VLLM_GPUS VLLM_SERVER_DEV_MODE=1 ${SERVE[*]}"
  echo "CUDA_VISIBLE_DEVICES=$TRAINER_GPUS ${LOOP[*]} [--weight-world-size <server world size + 1>]"
  exit 0
fi
VLLM_PID=""
cleanup() {
  if [ -n "$VLLM_PID" ] && kill -0 "$VLLM_PID" 2>/dev/null; then
    kill "$VLLM_PID" 2>/dev/null || true       # the server this script started, by its pid
    wait "$VLLM_PID" 2>/dev/null || true
  fi
}
trap cleanup EXIT
if [ "$BACKEND" = "http" ]; then
  CUDA_VISIBLE_DEVICES=$VLLM_GPUS VLLM_SERVER_DEV_MODE=1 "${SERVE[@]}" > "$VLLM_LOG" 2>&1 &
  VLLM_PID=$!
  ready=0
  for i in $(seq 1 "${VLLM_READY_RETRIES:-120}"); do
    if python -c "import sys, urllib.request; urllib.request.urlopen(sys.argv[1] + '/v1/models', timeout=5)" "$BASE_URL" 2>/dev/null; then
      ready=1; break
    fi
    if ! kill -0 "$VLLM_PID" 2>/dev/null; then tail -n 120 "$VLLM_LOG" || true; exit 1; fi
    sleep 2
  done
  [ "$ready" = "1" ] || { echo "vllm serve did not come up; see $VLLM_LOG" >&2; exit 1; }
  if [ "${STATIC_SPLIT:-0}" != "1" ]; then
    WS=$(python -m cverl_b200.cli.vllm_native_rl_control --base-url "$BASE_URL" world-size | python -c "import json, sys; print(json.load(sys.stdin)['world_size'])")
    LOOP+=(--weight-world-size "${WORLD_SIZE:-$((WS + 1))}")
  fi
fi
CUDA_VISIBLE_DEVICES=$TRAINER_GPUS "${LOOP[@]}"
