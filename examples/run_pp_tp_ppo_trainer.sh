#!/bin/bash
# The distributed PPO / GRPO / SFT trainer driven by environment variables (the variable names of the
# reference's launcher, tools/distributed/run_qwen_pp_tp_ppo_trainer.sh, so existing job files keep working).
# Every variable has a default; the model directory is the first argument (omit it for a built-in random shape,
# CONFIG=qwen3_5_0_8b | qwen3_30b_a3b | tiny | tiny_moe).  Extra arguments go to the trainer unchanged.
set -euo pipefail
MODEL_DIR=${1:-}; shift || true
DP_SIZE=${DP_SIZE:-1}; PP_SIZE=${PP_SIZE:-2}; CP_SIZE=${CP_SIZE:-1}; TP_SIZE=${TP_SIZE:-2}; EP_SIZE=${EP_SIZE:-1}
WORLD_SIZE=$((DP_SIZE * PP_SIZE * CP_SIZE * TP_SIZE * EP_SIZE))
ARGS=(--dp-size "$DP_SIZE" --pp-size "$PP_SIZE" --cp-size "$CP_SIZE" --tp-size "$TP_SIZE" --ep-size "$EP_SIZE"
      --layers "${LAYERS:--1}" --prompt-len "${PROMPT_LEN:-256}" --response-len "${RESPONSE_LEN:-1024}"
      --micro-batches "${MICRO_BATCHES:-$PP_SIZE}" --micro-batch-seqs "${MICRO_BATCH_SEQS:-1}"
      --grad-accum-steps "${GRAD_ACCUM_STEPS:-1}" --steps "${STEPS:-1}" --train-mode "${TRAIN_MODE:-ppo}"
      --lr "${LR:-1e-6}" --clip-ratio "${CLIP_RATIO:-0.2}" --max-grad-norm "${MAX_GRAD_NORM:-1.0}"
      --dp-grad-bucket-mb "${DP_GRAD_BUCKET_MB:-25}" --tp-grad-bucket-mb "${TP_GRAD_BUCKET_MB:-${DP_GRAD_BUCKET_MB:-25}}"
      --dp-grad-comm-dtype "${DP_GRAD_COMM_DTYPE:-model}" --tp-grad-comm-dtype "${TP_GRAD_COMM_DTYPE:-${DP_GRAD_COMM_DTYPE:-model}}"
      --advantage-scale "${ADVANTAGE_SCALE:-1.0}" --master-weights "${MASTER_WEIGHTS:-false}"
      --dp-shard-optimizer "${DP_SHARD_OPTIMIZER:-true}" --dp-flat-shard-optimizer "${DP_FLAT_SHARD_OPTIMIZER:-true}"
      --skip-optimizer-step "${SKIP_OPTIMIZER_STEP:-false}" --measure-param-delta "${MEASURE_PARAM_DELTA:-false}"
      --vary-tokens-by-step "${VARY_TOKENS_BY_STEP:-false}" --dtype "${DTYPE:-bfloat16}"
      --kl-coef "${KL_COEF:-0}" --zero-stage "${ZERO_STAGE:-1}" --zero-comm "${ZERO_COMM:-symm}"
      --tp-comm "${TP_COMM:-sp}" --ep-comm "${EP_COMM:-symm}" --cp-comm "${CP_COMM:-nccl}" --cp-attn "${CP_ATTN:-zigzag}")
[ -n "$MODEL_DIR" ] && ARGS+=(--model-dir "$MODEL_DIR") || ARGS+=(--config "${CONFIG:-qwen3_5_0_8b}")
[ -n "${JSONL_INPUT:-}" ] && ARGS+=(--jsonl-input "$JSONL_INPUT" --jsonl-max-examples "${JSONL_MAX_EXAMPLES:-16}")
[ -n "${TOKENIZER_JSON:-}" ] && ARGS+=(--tokenizer-json "$TOKENIZER_JSON")
[ -n "${ROLLOUT_JSON:-}" ] && ARGS+=(--rollout-json "$ROLLOUT_JSON")
[ -n "${ROLLOUT_DIR:-}" ] && ARGS+=(--rollout-dir "$ROLLOUT_DIR")
[ -n "${ROLLOUT_IPC_JSON:-}" ] && ARGS+=(--rollout-ipc-json "$ROLLOUT_IPC_JSON")
[ -n "${ROLLOUT_IPC_DIR:-}" ] && ARGS+=(--rollout-ipc-dir "$ROLLOUT_IPC_DIR")
if [ -n "${ROLLOUT_NCCL_ID_FILE:-}" ]; then
  ARGS+=(--rollout-nccl-id-file "$ROLLOUT_NCCL_ID_FILE" --rollout-nccl-world-size "${ROLLOUT_NCCL_WORLD_SIZE:-0}"
         --rollout-nccl-rank-offset "${ROLLOUT_NCCL_RANK_OFFSET:-0}" --rollout-nccl-source-rank "${ROLLOUT_NCCL_SOURCE_RANK:-0}")
fi
[ -n "${CHECKPOINT_DIR:-}" ] && ARGS+=(--checkpoint-dir "$CHECKPOINT_DIR" --checkpoint-every "${CHECKPOINT_EVERY:-1}")
[ -n "${RESUME_CHECKPOINT:-}" ] && ARGS+=(--resume-checkpoint "$RESUME_CHECKPOINT")
[ -n "${METRICS_CSV:-}" ] && ARGS+=(--metrics-csv "$METRICS_CSV")
[ -n "${NCCL_LIB_DIR:-}" ] && export LD_LIBRARY_PATH="$NCCL_LIB_DIR:${LD_LIBRARY_PATH:-}"
if [ -n "${MAX_RESTARTS:-}" ] || [ -n "${LOG_DIR:-}" ]; then
  # supervised: one log per rank under LOG_DIR, a failed or stalled rank ends the attempt, and the job is started
  # again from the newest complete checkpoint of CHECKPOINT_DIR up to MAX_RESTARTS times
  exec python -m cverl_b200.cli.launch --nproc "${LOCAL_WORLD_SIZE:-$WORLD_SIZE}" --master-addr 127.0.0.1 \
    --master-port "${MASTER_PORT:-29500}" --max-restarts "${MAX_RESTARTS:-0}" --log-dir "${LOG_DIR:-}" \
    --stall-timeout-s "${STALL_TIMEOUT_S:-0}" -- -m cverl_b200.trainer.ppo_trainer "${ARGS[@]}" "$@"
fi
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "${LOCAL_WORLD_SIZE:-$WORLD_SIZE}" \
  --master-addr 127.0.0.1 --master-port "${MASTER_PORT:-29500}" -m cverl_b200.trainer.ppo_trainer "${ARGS[@]}" "$@"
