#!/bin/bash
# Static trainer / rollout split on one node: the first TRAINERS ranks train (data parallel), the others generate;
# rollout batches travel GPU to GPU, new weights are pushed back after every step.  WEIGHT_PUSH = nccl (bucketed
# send / recv), symm (this package's peer-store kernel) or nvls (one multicast store through the NVSwitch).
# The reference's counterpart: examples/run_vllm_static_split_4gpu_h20.sh with its own rollout workers.
set -euo pipefail
GPUS=${GPUS:-4}; TRAINERS=${TRAINERS:-$((GPUS / 2))}
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 \
  -m cverl_b200.cli.static_split --backend nccl --trainers "$TRAINERS" --steps "${STEPS:-3}" \
  --weight-push "${WEIGHT_PUSH:-symm}" --policy "${POLICY:-tiny}" ${MODEL_DIR:+--model-dir "$MODEL_DIR"} "$@"
