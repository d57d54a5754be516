#!/bin/bash
# Multi-node launcher: one task per node under Slurm (srun --ntasks-per-node=1 this script).
#  * optional dataset staging to node-local disk with a .stage_complete sentinel (STAGE_DATA=1);
#  * rendezvous: MASTER_ADDR = first host of the allocation, MASTER_PORT = 20000 + job id % 20000,
#    published by node 0 through a file in LOGDIR and read by the other nodes;
#  * fabric sanity check before the run (exit 42 when no NVLink/IB device is visible);
#  * stale /dev/shm/nccl-* cleanup; per-trial SEED = ROOT_SEED + trial index.
# Mirrors flux1/primus/run_with_docker_slurm.sh:1-340 and recommendation_v4/hstu/run_with_docker_slurm.sh:55-216.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
: "${WORKLOAD:?}" "${DGXSYSTEM:?}"
: "${LOGDIR:=$(pwd)/results/${WORKLOAD}}"
: "${SLURM_JOB_ID:=0}" "${SLURM_NODEID:=0}" "${SLURM_JOB_NUM_NODES:=1}"
mkdir -p "${LOGDIR}"
export NNODES="${SLURM_JOB_NUM_NODES}" NODE_RANK="${SLURM_NODEID}"

if [ "${STAGE_DATA:-0}" = "1" ] && [ -n "${DATADIR:-}" ]; then
  LOCAL_DATA="${LOCAL_DATA_DIR:-/tmp/b200_train_data}/${WORKLOAD}"
  bash "${HERE}/stage_dataset_local.sh" "${DATADIR}" "${LOCAL_DATA}"
  export DATADIR="${LOCAL_DATA}"
fi

PORT_FILE="${LOGDIR}/.rendezvous_${SLURM_JOB_ID}"
if [ "${NODE_RANK}" = "0" ]; then
  MASTER_ADDR="$(scontrol show hostnames "${SLURM_JOB_NODELIST:-$(hostname)}" 2>/dev/null | head -n1 || hostname)"
  MASTER_PORT=$((20000 + SLURM_JOB_ID % 20000))
  echo "${MASTER_ADDR} ${MASTER_PORT}" > "${PORT_FILE}"
else
  for _ in $(seq 1 120); do [ -s "${PORT_FILE}" ] && break; sleep 1; done
  read -r MASTER_ADDR MASTER_PORT < "${PORT_FILE}"
fi
export MASTER_ADDR MASTER_PORT

# fabric pre-flight: at least one GPU and (multi-node) one InfiniBand / RoCE device
if ! nvidia-smi -L >/dev/null 2>&1; then echo "no GPU visible" >&2; exit 42; fi
if [ "${NNODES}" -gt 1 ] && [ -z "$(ls /sys/class/infiniband 2>/dev/null)" ]; then
  echo "multi-node run without an RDMA device" >&2; exit 42
fi
rm -f /dev/shm/nccl-* 2>/dev/null || true

exec bash "${HERE}/run_with_docker.sh"
