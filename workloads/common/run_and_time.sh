#!/bin/bash
# Timed run of one trial (inside the container, or on the host): banner, "STARTING TIMING RUN",
# the trainer under torchrun, "ENDING TIMING RUN" and the result line
#     RESULT,<benchmark>,,<seconds>,b200-train,<start date>
# With B200_QUIET=1 only :::MLLOG lines and these markers reach stdout.
# Contract of the reference's run_and_time.sh (small_llm_pretraining/primus/run_and_time.sh:52-75).
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REPO="$(cd "${HERE}/../.." && pwd)"
cd "${REPO}"
: "${WORKLOAD:?}"
: "${EXP:?EXP must name the experiment YAML (set by config_*.sh)}"
: "${TRAIN_MODE:=pretrain}"
: "${NGPU:=$(python -c 'import torch; print(max(torch.cuda.device_count(), 1))')}"
: "${NNODES:=1}"
: "${NODE_RANK:=0}"
: "${MASTER_ADDR:=127.0.0.1}"
: "${MASTER_PORT:=29500}"
: "${EXTRA_OVERRIDES:=}"

start=$(date +%s)
start_fmt=$(date +%Y-%m-%d\ %r)
echo "STARTING TIMING RUN AT ${start_fmt}"
echo "workload=${WORKLOAD} system=${DGXSYSTEM:-unknown} gpus=${NGPU} nodes=${NNODES} seed=${SEED:-0}"

set +e
if [ "${NGPU}" -gt 1 ] || [ "${NNODES}" -gt 1 ]; then
  python -m torch.distributed.run --nnodes="${NNODES}" --node-rank="${NODE_RANK}" --nproc-per-node="${NGPU}" \
    --master-addr "${MASTER_ADDR}" --master-port "${MASTER_PORT}" \
    -m mlperf_training_b200.trainer.cli "${TRAIN_MODE}" --config "${REPO}/workloads/${WORKLOAD}/${EXP}" ${EXTRA_OVERRIDES}
else
  python -m mlperf_training_b200.trainer.cli "${TRAIN_MODE}" --config "${REPO}/workloads/${WORKLOAD}/${EXP}" ${EXTRA_OVERRIDES}
fi
ret=$?
set -e

end=$(date +%s)
end_fmt=$(date +%Y-%m-%d\ %r)
echo "ENDING TIMING RUN AT ${end_fmt}"
echo "RESULT,${WORKLOAD},,$((end - start)),b200-train,${start_fmt}"
exit "${ret}"
