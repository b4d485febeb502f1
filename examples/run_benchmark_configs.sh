#!/bin/bash
# The five benchmark configurations of this repository through bench.py, on the GPUs of one node.
#   GPUS (default 8)  STEPS (default 5)  WARMUP (default 3)
set -euo pipefail
GPUS=${GPUS:-8}; STEPS=${STEPS:-5}; WARMUP=${WARMUP:-3}
RUN=(python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 bench.py --gpus "$GPUS"
     --steps "$STEPS" --warmup "$WARMUP")
python bench.py --config cpu_loss
"${RUN[@]}"                                   # Qwen3.5-0.8B GRPO actor update, DP x TP=2
"${RUN[@]}" --config moe30b_ep8_sft           # Qwen3-30B-A3B SFT, expert parallel over all GPUs
"${RUN[@]}" --config cp8_attention            # ring attention at 131,072 tokens + a 4-layer model step
"${RUN[@]}" --config zero2_dp8_push           # 30B ZeRO-2 step overlapped with backward + weight push
