#!/usr/bin/env bash
# launch.sh - one process per GPU.
#
#   ./launch.sh <plan_dir> [cmd...]        default cmd: python -m cai_b200.trainer
#
# Every process gets RANK / WORLD_SIZE / LOCAL_RANK and is handed its own plan.rankNNNNNN.bin plus
# the shared topology.bin (same contract as the reference's tools/launch.sh). Under SLURM the script
# is run once per task by srun; otherwise it starts one process per visible GPU (or a single CPU
# process running the analytic replay when there is no GPU).
set -euo pipefail

PLAN_DIR="${1:?usage: launch.sh <plan_dir> [cmd...]}"
shift || true
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
export MASTER_ADDR="${MASTER_ADDR:-127.0.0.1}"
export MASTER_PORT="${MASTER_PORT:-29555}"

run_rank() {  # $1 = rank, rest = command
  local rank="$1"; shift
  local plan
  plan="$(printf '%s/plan.rank%06d.bin' "$PLAN_DIR" "$rank")"
  RANK="$rank" "$@" "$plan" "$PLAN_DIR/topology.bin"
}

if [[ -n "${SLURM_PROCID:-}" ]]; then
  export WORLD_SIZE="${SLURM_NPROCS:?}" LOCAL_RANK="${SLURM_LOCALID:-0}"
  if [[ $# -eq 0 ]]; then set -- python -m cai_b200.trainer; fi
  cd "$HERE" && run_rank "$SLURM_PROCID" "$@"
  exit $?
fi

if command -v nvidia-smi >/dev/null 2>&1 && nvidia-smi -L >/dev/null 2>&1; then
  NGPU="$(nvidia-smi -L | wc -l)"
  if [[ $# -eq 0 ]]; then set -- python -m cai_b200.trainer; fi
else
  echo "no GPU visible: one CPU process, analytic replay" >&2
  NGPU=1
  if [[ $# -eq 0 ]]; then set -- "$HERE/bin/trainer"; fi
fi
export WORLD_SIZE="$NGPU"
pids=()
for ((g = 0; g < NGPU; g++)); do
  ( cd "$HERE" && LOCAL_RANK="$g" run_rank "$g" "$@" ) &
  pids+=("$!")
done
rc=0
for p in "${pids[@]}"; do wait "$p" || rc=$?; done
exit "$rc"
