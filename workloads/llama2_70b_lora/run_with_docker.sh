#!/bin/bash
# Launch surface of the llama2_70b_lora workload: see workloads/common/run_with_docker.sh for the contract.
export WORKLOAD=llama2_70b_lora
exec bash "$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)/../common/run_with_docker.sh" "$@"
