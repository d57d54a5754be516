#!/bin/bash
# Launch surface of the flux1 workload: see workloads/common/run_with_docker.sh for the contract.
export WORKLOAD=flux1
exec bash "$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)/../common/run_with_docker.sh" "$@"
