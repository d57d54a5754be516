#!/bin/bash
#SBATCH --job-name=b200-train
#SBATCH --nodes=1
#SBATCH --ntasks-per-node=1
#SBATCH --gpus-per-node=8
#SBATCH --exclusive
#SBATCH --time=04:00:00
# Slurm batch wrapper: sbatch --export=ALL,WORKLOAD=...,DGXSYSTEM=... workloads/common/job.sh
# Training from node-local data (STAGE_DATA=1) avoids the throughput loss of a network file system.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
srun --ntasks-per-node=1 bash "${HERE}/run_with_docker_slurm.sh"
