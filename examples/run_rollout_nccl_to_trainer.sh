#!/bin/bash
# A rollout-batch source process and the trainer joined by an NCCL communicator that is formed through an id file
# (no launcher in common): the source sends rollout batches (token ids, masks, old log-probs, advantages) from its
# GPU straight into the trainer's first stage.  The reference's pair: tools/distributed/run_rollout_nccl_to_pp_tp_ppo.sh.
#   TRAINER_GPUS (default 2: tp2)  SOURCE_GPU (default: the next one)  STEPS  PROMPT_LEN  RESPONSE_LEN
set -euo pipefail
MODEL_DIR=${1:-}; shift || true
TP_SIZE=${TP_SIZE:-2}; STEPS=${STEPS:-2}; PROMPT_LEN=${PROMPT_LEN:-64}; RESPONSE_LEN=${RESPONSE_LEN:-64}
ID_FILE=${ROLLOUT_NCCL_ID_FILE:-/tmp/cverl_b200_rollout_$$.id}
rm -f "$ID_FILE"
MODEL=(--config "${CONFIG:-qwen3_5_0_8b}"); [ -n "$MODEL_DIR" ] && MODEL=(--model-dir "$MODEL_DIR")
TARGETS=$(seq -s, 1 "$TP_SIZE")                      # the source is rank 0 of the joint communicator
CUDA_VISIBLE_DEVICES=${SOURCE_GPU:-$TP_SIZE} python -m cverl_b200.cli.rollout_batch_source --id-file "$ID_FILE" \
  --rank 0 --world-size $((TP_SIZE + 1)) --target-ranks "$TARGETS" --device cuda:0 --steps "$STEPS" \
  --batch "${BATCH:-4}" --prompt-len "$PROMPT_LEN" --response-len "$RESPONSE_LEN" --backend nccl &
SRC=$!
trap 'kill $SRC 2>/dev/null || true' EXIT
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$TP_SIZE" --master-addr 127.0.0.1 \
  -m cverl_b200.trainer.ppo_trainer --tp "$TP_SIZE" --steps "$STEPS" --prompt-len "$PROMPT_LEN" \
  --response-len "$RESPONSE_LEN" "${MODEL[@]}" --rollout-nccl-id-file "$ID_FILE" \
  --rollout-nccl-world-size $((TP_SIZE + 1)) --rollout-nccl-rank-offset 1 --rollout-nccl-source-rank 0 "$@"
wait $SRC
