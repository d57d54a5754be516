#!/bin/bash
# Launch surface of the hstu workload: see workloads/common/run_with_docker.sh for the contract.
export WORKLOAD=hstu
exec bash "$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)/../common/run_with_docker.sh" "$@"
