"""Worker for the failure-detection tests (CPU only).
  heartbeat <store_file> <rank> <world> : rank 1 stops beating after 3 steps and leaves; the others must notice.
  timeout   : under torchrun; rank 1 never joins the second all-reduce; rank 0's collective must end with an error."""
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.parallel import health  # noqa: E402


def heartbeat(path, rank, world):
    store = dist.FileStore(path, world)
    hb = health.Heartbeat(store, rank, world, interval_s=0.2).start()
    try:
        for step in range(200):
            if rank == 1 and step == 3:
                hb.stop()                       # the "failed" rank: leaves between steps, says nothing
                health.clean_exit(0)
            hb.check(timeout_s=1.5)             # before launching the step
            time.sleep(0.1)                     # the step
        print("no failure seen", flush=True)
        health.clean_exit(1)
    except health.RankFailure as e:
        print(f"rank {rank} detected {e.ranks}", flush=True)
        health.clean_exit(health.EXIT_RANK_FAILURE)


def timeout():
    rank = int(os.environ["RANK"])
    os.environ["PG_TIMEOUT_S"] = "3"
    dist.init_process_group("gloo", timeout=health.pg_timeout())
    t = torch.ones(4)
    dist.all_reduce(t)
    assert float(t[0]) == 2.0
    if rank == 1:
        time.sleep(8)                            # never joins the next collective
        health.clean_exit(0)
    try:
        dist.all_reduce(t)
    except Exception as e:                        # the watchdog timeout ended the collective
        print(f"rank 0 collective ended with {type(e).__name__}", flush=True)
        health.clean_exit(health.EXIT_RANK_FAILURE)
    health.clean_exit(1)


if __name__ == "__main__":
    if sys.argv[1] == "heartbeat":
        heartbeat(sys.argv[2], int(sys.argv[3]), int(sys.argv[4]))
    else:
        timeout()
