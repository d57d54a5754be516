#!/bin/bash
# Launch surface of the llama31_8b workload: see workloads/common/run_with_docker.sh for the contract.
export WORKLOAD=llama31_8b
exec bash "$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)/../common/run_with_docker.sh" "$@"
