#!/bin/bash
# ResNet-152 training-step throughput on CIFAR-10 tensors (the reference's examples/run_resnet152_cifar10_bench.sh
# with prepare_cifar10_hf.sh folded in).  With CIFAR10_PARQUET=<train parquet of the Hugging Face dataset> the
# images are first exported to tensors under DATA_DIR; without data the bench draws synthetic images.
#   [CIFAR10_PARQUET=train.parquet] [DATA_DIR=out] examples/run_resnet_cifar10_bench.sh [extra bench flags]
set -euo pipefail
DATA_DIR=${DATA_DIR:-}
if [ -n "${CIFAR10_PARQUET:-}" ]; then
  DATA_DIR=${DATA_DIR:-${TMPDIR:-/tmp}/cverl_b200_cifar10}
  python -m cverl_b200.cli.export_cifar10_tensors --parquet "$CIFAR10_PARQUET" --out-dir "$DATA_DIR" --split "${SPLIT:-train}"
fi
ARGS=(--steps "${STEPS:-20}" --warmup "${WARMUP:-5}" --batch-size "${BATCH_SIZE:-128}" --dtype "${DTYPE:-bfloat16}"
      --depth "${DEPTH:-152}")
[ -n "$DATA_DIR" ] && ARGS+=(--data-dir "$DATA_DIR")
[ -n "${DEVICE:-}" ] && ARGS+=(--device "$DEVICE")
[ "${CHANNELS_LAST:-0}" = "1" ] && ARGS+=(--channels-last)
exec python -m cverl_b200.cli.resnet_cifar10_bench "${ARGS[@]}" "$@"
