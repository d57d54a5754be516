"""Relaunch-based recovery: start the ranks of a run, and when the run stops on a failure start it again
so that it resumes from its last complete checkpoint.

    python -m mlperf_training_b200.trainer.supervisor --nproc 8 [--max-restarts 3] [--shrink --min-nproc 2] \\
        -- pretrain --config <experiment.yaml> [key=value ...]

Everything after ``--`` is handed to ``trainer.cli`` under ``torch.distributed.run`` (one node, rendezvous on
127.0.0.1).  Exit codes decide what happens next: 0 ends the job; 42 (fault injection after a
checkpoint) and 43 (a rank stopped answering: ``parallel.health.EXIT_RANK_FAILURE``) and any other
failure are restarted while restarts are left.  With ``--shrink`` a restart after a lost rank uses the next
smaller world size that divides the original one (the rank's GPU is taken to be gone); the resumed run
re-cuts the sharded optimizer state for its new size (``checkpoint/reshard.py``).  One JSON line per
launch goes to stdout.

The reference recovers the same way: crash-safe checkpoints and a relaunch by the launcher script or
the Slurm requeue, not in-job elasticity (generative_recommenders/dlrm_v4/checkpoint.py:338-525;
flux1/primus/run_with_docker_slurm.sh:218-261 exits 42 from its pre-flight for the same purpose).
"""
from __future__ import annotations

import argparse
import json
import os
import socket
import subprocess
import sys
import time

EXIT_INJECTED = 42
EXIT_RANK_FAILURE = 43


def next_world(current: int, original: int, min_world: int) -> int | None:
    """Largest world size below ``current`` that divides ``original`` and is at least ``min_world``."""
    for n in range(current - 1, max(min_world, 1) - 1, -1):
        if original % n == 0:
            return n
    return None


def decide(rc: int, restarts_done: int, max_restarts: int, world: int, original: int, min_world: int, shrink: bool) -> tuple[str, int]:
    """('done' | 'restart' | 'give_up', world size of the next launch)."""
    if rc == 0:
        return "done", world
    if restarts_done >= max_restarts:
        return "give_up", world
    if shrink and rc == EXIT_RANK_FAILURE:
        smaller = next_world(world, original, min_world)
        if smaller is None:
            return "give_up", world
        return "restart", smaller
    return "restart", world


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worst_rank_code(rc: int, log_text: str = "") -> int:
    """torchrun reports 1 for any failed child; the ranks' own codes are in its summary."""
    for code in (EXIT_RANK_FAILURE, EXIT_INJECTED):
        if f"exitcode: {code}" in log_text or f"exitcode  : {code}" in log_text:
            return code
    return rc


def supervise(world: int, cli_args: list[str], *, max_restarts: int = 3, shrink: bool = False, min_world: int = 1,
              env: dict | None = None, out=sys.stdout, run=None) -> int:
    """Returns the exit code of the last launch.  ``run(world, cli_args) -> exit code`` replaces the
    subprocess launch in tests."""
    original, restarts = world, 0
    while True:
        t0 = time.time()
        rc = run(world, cli_args) if run is not None else _launch_logged(world, cli_args, env)
        action, nxt = decide(rc, restarts, max_restarts, world, original, min_world, shrink)
        print(json.dumps({"supervisor": "launch_end", "world": world, "exit_code": rc, "seconds": round(time.time() - t0, 1),
                          "restarts": restarts, "action": action, "next_world": nxt}), file=out, flush=True)
        if action != "restart":
            return rc
        restarts, world = restarts + 1, nxt


def _launch_logged(world: int, cli_args: list[str], env: dict | None) -> int:
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), "-m", "mlperf_training_b200.trainer.cli", *cli_args]
    proc = subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    tail: list[str] = []
    for line in proc.stdout:
        sys.stdout.write(line)
        tail.append(line)
        del tail[:-400]
    return worst_rank_code(proc.wait(), "".join(tail))


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    usage = "usage: supervisor --nproc N [--max-restarts K] [--shrink --min-nproc M] -- <trainer.cli arguments>"
    if argv and argv[0] in ("-h", "--help"):
        print(usage)
        return 0
    if "--" not in argv:
        print(usage, file=sys.stderr)
        return 2
    cut = argv.index("--")
    ap = argparse.ArgumentParser(prog="b200-supervisor")
    ap.add_argument("--nproc", type=int, required=True)
    ap.add_argument("--max-restarts", type=int, default=3)
    ap.add_argument("--shrink", action="store_true")
    ap.add_argument("--min-nproc", type=int, default=1)
    args = ap.parse_args(argv[:cut])
    return supervise(args.nproc, argv[cut + 1:], max_restarts=args.max_restarts, shrink=args.shrink, min_world=args.min_nproc,
                     env=dict(os.environ))


if __name__ == "__main__":
    sys.exit(main())
