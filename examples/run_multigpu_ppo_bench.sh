#!/bin/bash
# Whole-run wall-clock throughput of two 4-rank layouts of the distributed trainer (PP2 x TP2 and PP4 x TP1) on a
# few layers and very short sequences: process start, model construction and the steps are all inside the timed
# span, so this measures launch overhead as much as the step (the harness of the reference's
# tools/bench/qwen_multigpu_ppo_bench.sh).  For steady-state step throughput use bench.py.
#   examples/run_multigpu_ppo_bench.sh [MODEL_DIR] [extra trainer flags, e.g. --backend gloo --dtype float32]
# Writes $OUT_DIR/multigpu_ppo_bench.csv (case,pp,tp,micro_batches,steps,layers,dtype,seconds,steps_per_second,
# tokens_per_second,log) and prints it.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
MODEL_DIR=${1:-}; shift || true
OUT_DIR=${OUT_DIR:-${TMPDIR:-/tmp}/cverl_b200_bench}
OUT_CSV=${OUT_CSV:-$OUT_DIR/multigpu_ppo_bench.csv}
export LAYERS=${LAYERS:-4} PROMPT_LEN=${PROMPT_LEN:-2} RESPONSE_LEN=${RESPONSE_LEN:-2} STEPS=${STEPS:-5}
export DTYPE=${DTYPE:-bfloat16} ADVANTAGE_SCALE=${ADVANTAGE_SCALE:-0.05} LR=${LR:-1e-10} DP_SIZE=1 CP_SIZE=1 EP_SIZE=1
export TP_COMM=${TP_COMM:-nccl} ZERO_COMM=${ZERO_COMM:-nccl} EP_COMM=nccl CP_COMM=nccl   # rows too short for the peer paths
mkdir -p "$OUT_DIR"
echo "case,pp,tp,micro_batches,steps,layers,dtype,seconds,steps_per_second,tokens_per_second,log" > "$OUT_CSV"
port=${MASTER_PORT:-29540}
run_case() {
  local name=$1 pp=$2 tp=$3 mb=$4 log="$OUT_DIR/$1.bench.log"
  local t0 t1
  shift 4
  t0=$(date +%s%N)
  PP_SIZE=$pp TP_SIZE=$tp MICRO_BATCHES=$mb MASTER_PORT=$port "$HERE/run_pp_tp_ppo_trainer.sh" "$MODEL_DIR" "$@" | tee "$log"
  t1=$(date +%s%N)
  port=$((port + 1))
  if grep -Eiq '=(nan|-?inf)( |$)' "$log"; then echo "$name produced non-finite values" >&2; exit 1; fi
  if ! grep -q "^step=$((STEPS - 1)) " "$log"; then echo "$name did not reach step $((STEPS - 1))" >&2; exit 1; fi
  awk -v n="$name" -v pp="$pp" -v tp="$tp" -v mb="$mb" -v st="$STEPS" -v ly="$LAYERS" -v dt="$DTYPE" -v s="$t0" -v e="$t1" \
      -v tok=$((STEPS * mb * (PROMPT_LEN + RESPONSE_LEN))) -v lg="$log" \
      'BEGIN { sec = (e - s) / 1e9; printf "%s,%d,%d,%d,%d,%d,%s,%.6f,%.6f,%.6f,%s\n", n, pp, tp, mb, st, ly, dt, sec, st / sec, tok / sec, lg }' >> "$OUT_CSV"
}
run_case qwen_pp2_tp2_ppo 2 2 2 "$@"
run_case qwen_pp4_tp1_ppo 4 1 4 "$@"
cat "$OUT_CSV"
