#!/bin/bash
# Fails (exit 1) when any local GPU already holds memory or runs a compute process.
set -euo pipefail
busy=0
while IFS=, read -r idx used; do
  used="${used// /}"
  if [ "${used:-0}" -gt 1024 ]; then echo "GPU ${idx} has ${used} MiB in use"; busy=1; fi
done < <(nvidia-smi --query-gpu=index,memory.used --format=csv,noheader,nounits)
if [ -n "$(nvidia-smi --query-compute-apps=pid --format=csv,noheader 2>/dev/null)" ]; then
  echo "compute processes are running"; busy=1
fi
exit "${busy}"
