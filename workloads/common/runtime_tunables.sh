#!/bin/bash
# Host tuning before the trials (best effort; every step is skipped without the privilege):
# drop the page cache, performance governor, NUMA balancing off, transparent huge pages on.
# GPU clocks, power limits and persistence mode are deliberately left untouched.
sync
(echo 3 > /proc/sys/vm/drop_caches) 2>/dev/null || true
command -v cpupower >/dev/null 2>&1 && cpupower frequency-set -g performance >/dev/null 2>&1 || true
(echo 0 > /proc/sys/kernel/numa_balancing) 2>/dev/null || true
(echo always > /sys/kernel/mm/transparent_hugepage/enabled) 2>/dev/null || true
exit 0
