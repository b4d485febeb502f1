#!/bin/bash
# Multi-process smokes on GPUs (use --backend gloo to run them on CPU).
set -euo pipefail
for spec in "tp 2" "dp_tp 4" "pp_tp 4"; do
  set -- $spec
  python -m torch.distributed.run --nnodes=1 --nproc-per-node "$2" --master-addr 127.0.0.1 \
    -m cverl_b200.cli.parallel_smoke --mode "$1" "${@:3}"
done
