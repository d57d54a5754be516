"""Failure detection on the host: heartbeats through a key-value store, straggler detection,
timed barriers, process-group timeout, clean hard exit.

Recovery is relaunch-based, as in the reference: a run that loses a rank stops, the supervisor
(``run_with_docker.sh`` / Slurm requeue) starts it again and it resumes from the last complete
checkpoint (generative_recommenders/dlrm_v4/checkpoint.py:338-525).  What this module adds is that
the surviving ranks *notice* on the host, between steps, instead of hanging in their next
collective:

* ``Heartbeat``       every rank bumps ``hb/<rank>`` in a ``torch.distributed`` store from a daemon
                      thread; ``stale(timeout)`` lists ranks whose counter has not moved.  A trainer
                      calls ``check()`` before it launches a step and gets ``RankFailure``.
                      ``arrive(step, timeout)`` is the stricter form: a store rendezvous before every
                      step, so a rank that left is noticed before anything is launched.
* ``pg_timeout()``    the watchdog timeout handed to ``init_process_group`` (``PG_TIMEOUT_S``;
                      generative_recommenders/dlrm_v4/train/utils.py:236-268), so a collective whose peer is gone ends with an error.
* ``timed_barrier``   a barrier that reports how long it waited and warns above a threshold
                      (window-boundary skew absorption, utils.py:356-402).
* ``StragglerDetector``  per-rank step times, all-gathered every ``interval`` steps; ranks slower
                      than ``factor`` x median are reported (Megatron / NVRx straggler detection is
                      wired but disabled in the reference: llama2_sft/primus/src/llama2_custom.py:1394-1418).
* ``clean_exit``      flush and ``os._exit`` so library finalisers cannot abort after a failure
                      (generative_recommenders/dlrm_v4/clean_exit.py).

No part of this touches a GPU: failures are injected and detected on the host.
"""
from __future__ import annotations

import datetime
import os
import sys
import threading
import time

import torch
import torch.distributed as dist

EXIT_RANK_FAILURE = 43


class RankFailure(RuntimeError):
    def __init__(self, ranks: list[int], waited_s: float):
        super().__init__(f"no heartbeat from rank(s) {ranks} for {waited_s:.1f} s")
        self.ranks = ranks


def pg_timeout(default_s: float = 600.0) -> datetime.timedelta:
    return datetime.timedelta(seconds=float(os.environ.get("PG_TIMEOUT_S", default_s)))


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval_s: float = 1.0, prefix: str = "hb"):
        self.store, self.rank, self.world, self.interval, self.prefix = store, rank, world, interval_s, prefix
        self._stop = threading.Event()
        self._thread = None
        self._seen: dict[int, tuple[int, float]] = {}
        self.beats = 0

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self) -> None:
        self.beats += 1
        self.store.set(self._key(self.rank), str(self.beats))

    def start(self) -> "Heartbeat":
        self.beat()

        def loop():
            while not self._stop.wait(self.interval):
                try:
                    self.beat()
                except Exception:       # the store is gone: the job is ending
                    return
        self._thread = threading.Thread(target=loop, name="heartbeat", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)

    def stale(self, timeout_s: float) -> list[int]:
        """Ranks whose counter did not change for ``timeout_s`` (as observed by this rank)."""
        now, out = time.monotonic(), []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                v = int(self.store.get(self._key(r)).decode()) if self.store.check([self._key(r)]) else -1
            except Exception:
                v = -1
            last = self._seen.get(r)
            if last is None or last[0] != v:
                self._seen[r] = (v, now)
            elif now - last[1] > timeout_s:
                out.append(r)
        return out

    def check(self, timeout_s: float) -> None:
        bad = self.stale(timeout_s)
        if bad:
            raise RankFailure(bad, timeout_s)

    def arrive(self, step: int, timeout_s: float, poll_s: float = 0.02) -> None:
        """Host-side rendezvous before a step is launched: publish that this rank is about to run
        ``step`` and wait until every rank has published the same (or a later) step.  A rank that
        left between steps never publishes, so the others raise ``RankFailure`` after ``timeout_s``
        with none of their kernels or collectives in flight."""
        self.store.set(f"{self.prefix}/at/{self.rank}", str(step))
        deadline = time.monotonic() + timeout_s
        waiting = [r for r in range(self.world) if r != self.rank]
        while waiting:
            still = []
            for r in waiting:
                key = f"{self.prefix}/at/{r}"
                try:
                    there = self.store.check([key]) and int(self.store.get(key).decode()) >= step
                except Exception:
                    there = False
                if not there:
                    still.append(r)
            waiting = still
            if waiting:
                if time.monotonic() > deadline:
                    raise RankFailure(waiting, timeout_s)
                time.sleep(poll_s)


def timed_barrier(group=None, warn_after_s: float = 5.0, label: str = "barrier", out=sys.stderr) -> float:
    t0 = time.perf_counter()
    if dist.is_available() and dist.is_initialized():
        dist.barrier(group=group)
    waited = time.perf_counter() - t0
    if waited > warn_after_s:
        print(f"[{label}] waited {waited:.1f} s for the slowest rank", file=out, flush=True)
    return waited


class StragglerDetector:
    def __init__(self, interval: int = 50, factor: float = 1.5, group=None):
        self.interval, self.factor, self.group = interval, factor, group
        self.times: list[float] = []
        self.reports: list[dict] = []

    def record(self, step_seconds: float) -> dict | None:
        self.times.append(step_seconds)
        if len(self.times) < self.interval:
            return None
        mine = torch.tensor([sum(self.times) / len(self.times)], dtype=torch.float64)
        self.times.clear()
        world = dist.get_world_size(self.group) if (dist.is_available() and dist.is_initialized()) else 1
        if world > 1:
            if dist.get_backend(self.group) == "nccl":
                mine = mine.cuda()
            allt = [torch.zeros_like(mine) for _ in range(world)]
            dist.all_gather(allt, mine, group=self.group)
            vals = [float(t) for t in allt]
        else:
            vals = [float(mine)]
        med = sorted(vals)[len(vals) // 2]
        rep = {"mean_step_s": vals, "median": med, "stragglers": [r for r, v in enumerate(vals) if v > self.factor * med]}
        self.reports.append(rep)
        return rep


def clean_exit(code: int) -> None:
    try:
        sys.stdout.flush()
        sys.stderr.flush()
    finally:
        os._exit(code)
