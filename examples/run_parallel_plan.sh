#!/bin/bash
# Prints the layout of a DP x PP x CP x TP x EP job (native planner binary).
set -euo pipefail
if [ $# -eq 0 ]; then set -- --dp 2 --pp 2 --tp 2 --layers 24 --micro-batches 4; fi
exec "$(dirname "$0")/../cverl_b200/lib/cverl_parallel_plan" "$@"
