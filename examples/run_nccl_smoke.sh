#!/bin/bash
# Every collective of the native NCCL communicator checked on WORLD_SIZE GPUs: one process per rank, rendezvous
# through an id file, one log per rank (the reference's tools/distributed/run_nccl_smoke.sh).
#   WORLD_SIZE=4 examples/run_nccl_smoke.sh            # native communicator (nccl/nccl_backend.cc)
#   BACKEND=torch CPU=1 WORLD_SIZE=2 examples/run_nccl_smoke.sh   # torch.distributed on gloo, no GPU
set -euo pipefail
WORLD_SIZE=${WORLD_SIZE:-4}
LOG_DIR=${LOG_DIR:-${TMPDIR:-/tmp}/cverl_b200_nccl_smoke}
ID_FILE=${ID_FILE:-$LOG_DIR/nccl_unique_id.bin}
mkdir -p "$LOG_DIR"
[ -e "$ID_FILE" ] && unlink "$ID_FILE"
[ -n "${NCCL_LIB_DIR:-}" ] && export LD_LIBRARY_PATH="$NCCL_LIB_DIR:${LD_LIBRARY_PATH:-}"
ARGS=(--backend "${BACKEND:-native}" --id-file "$ID_FILE")
[ "${CPU:-0}" = "1" ] && ARGS+=(--cpu)
[ "${SYNC_AFTER_OP:-0}" = "1" ] && ARGS+=(--sync-after-op)
exec python -m cverl_b200.cli.launch --nproc "$WORLD_SIZE" --master-port "${MASTER_PORT:-29530}" --log-dir "$LOG_DIR" \
  --grace-s 5 --attempt-timeout-s "${TIMEOUT_S:-300}" -- -m cverl_b200.cli.collectives_smoke "${ARGS[@]}"
