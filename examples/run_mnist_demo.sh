#!/bin/bash
# A small CNN trained on MNIST IDX files with Fp32MasterAdamW (the reference's examples/run_mnist_gpu_demo.sh).
#   examples/run_mnist_demo.sh [DATA_DIR with train-images-idx3-ubyte ... | omit for a synthetic ten-class problem]
set -euo pipefail
DATA_DIR=${1:-}; shift || true
ARGS=(--epochs "${EPOCHS:-1}" --batch-size "${BATCH_SIZE:-256}" --lr "${LR:-1e-3}")
[ -n "${METRICS_CSV:-}" ] && ARGS+=(--metrics-csv "$METRICS_CSV")
[ -n "${DEVICE:-}" ] && ARGS+=(--device "$DEVICE")
if [ -n "$DATA_DIR" ]; then ARGS+=(--data-dir "$DATA_DIR"); else ARGS+=(--synthetic); fi
exec python -m cverl_b200.cli.mnist_demo "${ARGS[@]}" "$@"
