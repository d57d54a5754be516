#!/bin/bash
# Host tuning before the trials (best effort; every step is skipped without the privilege):
# drop the page cache, performance governor, NUMA balancing off, transparent huge pages on.
# GPU clocks, power limits and persistence mode are deliberately left untouched.
# Off by default: the host belongs to its operator.  APPLY_HOST_TUNABLES=1 opts in.
if [ "${APPLY_HOST_TUNABLES:-0}" != "1" ]; then
  echo "runtime_tunables: host settings left as they are (set APPLY_HOST_TUNABLES=1 to apply them)"
  exit 0
fi
sync
(echo 3 > /proc/sys/vm/drop_caches) 2>/dev/null || true
command -v cpupower >/dev/null 2>&1 && cpupower frequency-set -g performance >/dev/null 2>&1 || true
(echo 0 > /proc/sys/kernel/numa_balancing) 2>/dev/null || true
(echo always > /sys/kernel/mm/transparent_hugepage/enabled) 2>/dev/null || true
exit 0
