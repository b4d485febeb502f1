#!/bin/bash
# Fused compute + collective kernels against NCCL on N GPUs of one node (default 8): ZeRO reduce-scatter + norm,
# AdamW + all-gather, GEMM + all-reduce, weight push.  One JSON line per case.
set -euo pipefail
N=${1:-8}; shift || true
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$N" --master-addr 127.0.0.1 \
  -m cverl_b200.bench_collectives "$@"
