#!/bin/bash
# Single-box launcher (one node, all local GPUs).
#
#   DGXSYSTEM=B200_1x8x1 [CONT=<image>] [DATADIR=...] [LOGDIR=...] [NEXP=1] [SEED=...] \
#       workloads/<workload>/run_with_docker.sh
#
# * validates the required variables and loads workloads/<workload>/config_${DGXSYSTEM}.sh as
#   DEFAULTS: a variable that is already set in the environment wins over the file;
# * with CONT set, starts a detached container with the data / log / code mounts and runs the
#   trials inside it (docker exec); without CONT the trials run directly on the host;
# * runs runtime_tunables.sh once, then NEXP trials, each with its own SEED and log file
#   ${LOGDIR}/${DATESTAMP}_${i}.log, and checks every trial log for MLLOG compliance.
#
# Same contract as the reference launchers (small_llm_pretraining/primus/run_with_docker.sh:10-155).
set -euo pipefail

HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REPO="$(cd "${HERE}/../.." && pwd)"
: "${WORKLOAD:?WORKLOAD must name a directory under workloads/}"
: "${DGXSYSTEM:?DGXSYSTEM must be set (e.g. B200_1x8x1)}"
WDIR="${REPO}/workloads/${WORKLOAD}"
CONFIG_FILE="${WDIR}/config_${DGXSYSTEM}.sh"
[ -f "${CONFIG_FILE}" ] || { echo "missing ${CONFIG_FILE}" >&2; exit 1; }

# a system file may pull in a file of shared settings (source ".../config_common.sh"): the files to read, in order
CONFIG_FILES=()
_collect_config_files() {
  local line inc
  while IFS= read -r line; do
    if [[ "${line}" =~ ^[[:space:]]*(source|\.)[[:space:]].*[/\"]([A-Za-z0-9_.-]+\.sh)\"?[[:space:]]*$ ]]; then
      inc="$(dirname "$1")/${BASH_REMATCH[2]}"
      [ -f "${inc}" ] && _collect_config_files "${inc}"
    fi
  done < "$1"
  CONFIG_FILES+=("$1")
}
_collect_config_files "${CONFIG_FILE}"

# config values are defaults: keep anything the caller already exported.  A later file (the system file) overrides an
# earlier one (the shared settings), as it would when sourced.
_apply_config_defaults() {
  local line key f
  declare -A from_caller=()
  for f in "${CONFIG_FILES[@]}"; do
    while IFS= read -r line; do
      [[ "${line}" =~ ^[[:space:]]*(export[[:space:]]+)?([A-Za-z_][A-Za-z0-9_]*)=(.*)$ ]] || continue
      key="${BASH_REMATCH[2]}"
      if [ -z "${from_caller[${key}]+x}" ]; then
        if [ -n "${!key+x}" ] && [ -z "${_set_by_config[${key}]+x}" ]; then from_caller[${key}]=1; continue; fi
        eval "export ${key}=${BASH_REMATCH[3]}"
        _set_by_config[${key}]=1
      fi
    done < "${f}"
  done
}
declare -A _set_by_config=()
_apply_config_defaults

: "${NEXP:=1}"
: "${LOGDIR:=${REPO}/results/${WORKLOAD}}"
: "${DATADIR:=}"
: "${DATESTAMP:=$(date +'%y%m%d%H%M%S')}"
: "${ROOT_SEED:=${SEED:-$RANDOM}}"
: "${CONT:=}"
: "${CONT_NAME:=b200_train_${WORKLOAD}}"
mkdir -p "${LOGDIR}"

run_in() {  # run a command on the host or inside the container
  if [ -n "${CONT}" ]; then
    docker exec "${_env_args[@]}" "${CONT_NAME}" "$@"
  else
    "$@"
  fi
}

_env_args=()
if [ -n "${CONT}" ]; then
  # forward every variable the config file names plus the launcher's own
  for _f in "${CONFIG_FILES[@]}"; do
    while IFS= read -r line; do
      [[ "${line}" =~ ^[[:space:]]*(export[[:space:]]+)?([A-Za-z_][A-Za-z0-9_]*)= ]] && _env_args+=("-e" "${BASH_REMATCH[2]}")
    done < "${_f}"
  done
  _env_args+=(-e WORKLOAD -e DGXSYSTEM -e SEED -e LOGDIR=/results -e DATADIR=/data)
  docker rm -f "${CONT_NAME}" >/dev/null 2>&1 || true
  docker run --gpus all --rm --detach --name "${CONT_NAME}" --ipc=host --ulimit memlock=-1 --ulimit stack=67108864 \
    ${DATADIR:+-v "${DATADIR}:/data"} -v "${LOGDIR}:/results" -v "${REPO}:/workspace/code" -w /workspace/code \
    "${CONT}" sleep infinity
  trap 'docker rm -f "${CONT_NAME}" >/dev/null 2>&1 || true' EXIT
fi

run_in bash "${HERE}/runtime_tunables.sh" || true

status=0
for i in $(seq 1 "${NEXP}"); do
  export SEED=$((ROOT_SEED + i - 1))
  LOG="${LOGDIR}/${DATESTAMP}_${i}.log"
  echo "Beginning trial ${i} of ${NEXP} (seed ${SEED})"
  # MLPerf asks for a cold page cache per trial; like the other host settings this is opt-in
  if [ "${APPLY_HOST_TUNABLES:-0}" = "1" ]; then sync && (echo 3 > /proc/sys/vm/drop_caches) 2>/dev/null || true; fi
  set +e
  run_in bash "${HERE}/run_and_time.sh" 2>&1 | tee "${LOG}"
  rc=${PIPESTATUS[0]}
  set -e
  [ "${rc}" -eq 0 ] || status="${rc}"
  python -m mlperf_training_b200.mllog.compliance "${LOG}" || status=1
done
exit "${status}"
