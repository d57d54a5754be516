#!/bin/bash
# Launch surface of the gpt_oss_20b workload: see workloads/common/run_with_docker.sh for the contract.
export WORKLOAD=gpt_oss_20b
exec bash "$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)/../common/run_with_docker.sh" "$@"
