#!/bin/bash
# Multi-rank regression of the distributed trainer: four 4-rank layouts x STEPS steps, each passing only if the log
# holds no nan / inf, the last step was reached, every rank saw a gradient and every rank's parameters moved
# (the checks of the reference's tools/distributed/run_qwen_multigpu_regression.sh:42-122).
#   examples/run_multigpu_regression.sh [MODEL_DIR] [extra trainer flags, e.g. --backend gloo]
# RUN_BASIC_TESTS=1 first runs the optimizer, topology and collective unit tests.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
MODEL_DIR=${1:-}; shift || true
OUT_DIR=${OUT_DIR:-${TMPDIR:-/tmp}/cverl_b200_regression}
export LAYERS=${LAYERS:-4} PROMPT_LEN=${PROMPT_LEN:-2} RESPONSE_LEN=${RESPONSE_LEN:-2} STEPS=${STEPS:-5}
export DTYPE=${DTYPE:-bfloat16} ADVANTAGE_SCALE=${ADVANTAGE_SCALE:-0.05} LR=${LR:-1e-4} CP_SIZE=1 EP_SIZE=1
export MEASURE_PARAM_DELTA=true TP_COMM=${TP_COMM:-nccl} ZERO_COMM=${ZERO_COMM:-nccl} EP_COMM=nccl CP_COMM=nccl
mkdir -p "$OUT_DIR"
if [ "${RUN_BASIC_TESTS:-0}" = "1" ]; then
  (cd "$HERE/.." && python -m pytest -q -m "not gpu" tests/test_topology_pipeline.py tests/test_core_algos_cpu.py \
      tests/test_parallel_cpu.py -k "topology or adamw or zero or collectives or pipeline") | tee "$OUT_DIR/basic_tests.log"
fi
port=${MASTER_PORT:-29560}
run_case() {
  local name=$1 dp=$2 pp=$3 tp=$4 mb=$5 shard=$6 log="$OUT_DIR/$1.log"
  shift 6
  echo "running $name: DP=$dp PP=$pp TP=$tp micro_batches=$mb dp_shard_optimizer=$shard steps=$STEPS"
  DP_SIZE=$dp PP_SIZE=$pp TP_SIZE=$tp MICRO_BATCHES=$mb DP_SHARD_OPTIMIZER=$shard DP_FLAT_SHARD_OPTIMIZER=$shard \
    MASTER_PORT=$port "$HERE/run_pp_tp_ppo_trainer.sh" "$MODEL_DIR" "$@" | tee "$log"
  port=$((port + 1))
  if grep -Eiq '=(nan|-?inf)( |$)' "$log"; then echo "$name produced non-finite values" >&2; exit 1; fi
  grep -q "^step=$((STEPS - 1)) " "$log" || { echo "$name did not reach step $((STEPS - 1))" >&2; exit 1; }
  if grep "^step=" "$log" | grep -vq "all_ranks_have_grad=true"; then echo "$name: a rank had no gradient" >&2; exit 1; fi
  if grep "^step=" "$log" | grep -vq "all_ranks_updated=true"; then echo "$name: a rank was not updated" >&2; exit 1; fi
}
run_case qwen_pp2_tp2_ppo 1 2 2 2 false "$@"
run_case qwen_pp4_tp1_ppo 1 4 1 4 false "$@"
run_case qwen_dp2_pp1_tp2_ppo 2 1 2 1 false "$@"
run_case qwen_dp2_pp1_tp2_sharded_optim 2 1 2 1 true "$@"
echo "multi-GPU PPO regression passed"
