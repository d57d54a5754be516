"""MLPerf ``:::MLLOG`` event stream, throughput timer and a minimal compliance check.

One JSON object per line, prefixed ``:::MLLOG``, with ``namespace, time_ms, event_type
(INTERVAL_START | INTERVAL_END | POINT_IN_TIME), key, value, metadata``.  Rank 0 writes; the other
ranks only take part in the optional barrier that aligns time stamps.  Event keys and their order
follow what the reference emits (primus_mllog/mlperf_pre_training.py:28-309 in the bundled wheel,
generative_recommenders/dlrm_v4/train/mlperf_logging_utils.py:62-352,660-835):
``cache_clear, init_start, submission_*, hyper-parameters, init_stop, run_start, epoch_start,
block_start/stop, eval_start/accuracy/stop, train_loss, tracked_stats, run_stop{status},
run_duration, overall_throughput``.
"""
from __future__ import annotations

import json
import os
import sys
import time
from typing import Any, Callable, TextIO

PREFIX = ":::MLLOG"

# event keys
CACHE_CLEAR = "cache_clear"
INIT_START, INIT_STOP = "init_start", "init_stop"
RUN_START, RUN_STOP = "run_start", "run_stop"
EPOCH_START, EPOCH_STOP = "epoch_start", "epoch_stop"
BLOCK_START, BLOCK_STOP = "block_start", "block_stop"
EVAL_START, EVAL_STOP, EVAL_ACCURACY = "eval_start", "eval_stop", "eval_accuracy"
TRAIN_LOSS = "train_loss"
TRACKED_STATS = "tracked_stats"
RUN_DURATION = "run_duration"
OVERALL_THROUGHPUT = "overall_throughput"
SUBMISSION_BENCHMARK, SUBMISSION_ORG = "submission_benchmark", "submission_org"
SUBMISSION_DIVISION, SUBMISSION_STATUS, SUBMISSION_PLATFORM = "submission_division", "submission_status", "submission_platform"
GLOBAL_BATCH_SIZE, SEED = "global_batch_size", "seed"
SUCCESS, ABORTED = "success", "aborted"

HYPERPARAMETER_KEYS = (
    "global_batch_size", "seed", "opt_base_learning_rate", "opt_learning_rate_warmup_steps",
    "opt_learning_rate_decay_steps", "opt_learning_rate_decay_schedule", "opt_adamw_beta_1", "opt_adamw_beta_2",
    "opt_adamw_epsilon", "opt_adamw_weight_decay", "opt_gradient_clip_norm", "gradient_accumulation_steps",
    "max_sequence_length", "eval_samples", "train_samples", "lora_rank", "lora_alpha",
)


class MLLogger:
    """Rank-0-gated writer of ``:::MLLOG`` lines.

    ``sync`` (a callable, normally ``torch.distributed.barrier``) is invoked on every rank before
    an event logged with ``sync=True`` so the time stamp means "all ranks reached this point".
    ``pre_emit_hook`` runs on rank 0 just before a line is written (used to flush a deferred
    train-loss read)."""

    def __init__(self, rank: int = 0, stream: TextIO | None = None, filename: str | None = None,
                 namespace: str = "", sync: Callable[[], None] | None = None, append: bool = False,
                 clock: Callable[[], float] = time.time):
        self.rank = rank
        self.stream = stream if stream is not None else sys.stdout
        self.file = open(filename, "a" if append else "w") if (filename and rank == 0) else None
        self.namespace = namespace
        self._sync = sync
        self.clock = clock
        self.pre_emit_hook: Callable[[], None] | None = None
        self.lines: list[dict] = []

    def _emit(self, event_type: str, key: str, value: Any, metadata: dict | None, sync: bool) -> None:
        if sync and self._sync is not None:
            self._sync()
        if self.rank != 0:
            return
        if self.pre_emit_hook is not None:
            hook, self.pre_emit_hook = self.pre_emit_hook, None
            try:
                hook()
            finally:
                self.pre_emit_hook = hook
        rec = {"namespace": self.namespace, "time_ms": int(self.clock() * 1000), "event_type": event_type,
               "key": key, "value": value, "metadata": metadata or {}}
        self.lines.append(rec)
        text = f"{PREFIX} {json.dumps(rec)}"
        print(text, file=self.stream, flush=True)
        if self.file is not None:
            print(text, file=self.file, flush=True)

    def event(self, key: str, value: Any = None, metadata: dict | None = None, sync: bool = False) -> None:
        self._emit("POINT_IN_TIME", key, value, metadata, sync)

    def start(self, key: str, value: Any = None, metadata: dict | None = None, sync: bool = False) -> None:
        self._emit("INTERVAL_START", key, value, metadata, sync)

    def end(self, key: str, value: Any = None, metadata: dict | None = None, sync: bool = False) -> None:
        self._emit("INTERVAL_END", key, value, metadata, sync)

    # ------------------------------------------------------------------ lifecycle helpers
    def log_init_start(self) -> None:
        self.event(CACHE_CLEAR, True)
        self.start(INIT_START)

    def log_submission(self, benchmark: str, org: str = "b200-train", platform: str = "1xB200x8",
                       division: str = "closed", status: str = "onprem") -> None:
        # MLLOG_SUBMISSION_* from the system config file win over the caller's defaults
        env = os.environ
        self.event(SUBMISSION_BENCHMARK, env.get("MLLOG_SUBMISSION_BENCHMARK", benchmark))
        self.event(SUBMISSION_ORG, env.get("MLLOG_SUBMISSION_ORG", org))
        self.event(SUBMISSION_DIVISION, env.get("MLLOG_SUBMISSION_DIVISION", division))
        self.event(SUBMISSION_STATUS, env.get("MLLOG_SUBMISSION_STATUS", status))
        self.event(SUBMISSION_PLATFORM, env.get("MLLOG_SUBMISSION_PLATFORM", platform))

    def log_hyperparameters(self, params: dict, env: dict | None = None) -> None:
        """Known MLPerf hyper-parameter keys from ``params``; ``MLLOG_<KEY>`` environment variables
        override or add values (the reference's ``extract`` of Megatron args + ``MLLOG_*`` env)."""
        env = os.environ if env is None else env
        merged = {k: v for k, v in params.items() if k in HYPERPARAMETER_KEYS}
        for k, v in env.items():
            if k.startswith("MLLOG_") and k[6:].lower() in HYPERPARAMETER_KEYS:
                merged[k[6:].lower()] = _num(v)
        for k in HYPERPARAMETER_KEYS:
            if k in merged:
                self.event(k, merged[k])

    def log_init_stop_run_start(self) -> None:
        self.end(INIT_STOP, sync=True)
        self.start(RUN_START, sync=True)

    def log_run_stop(self, success: bool, samples: int | None = None, duration_s: float | None = None) -> None:
        self.end(RUN_STOP, metadata={"status": SUCCESS if success else ABORTED}, sync=True)
        if duration_s is not None:
            self.event(RUN_DURATION, duration_s)
            if samples is not None and duration_s > 0:
                self.event(OVERALL_THROUGHPUT, samples / duration_s)

    def close(self) -> None:
        if self.file is not None:
            self.file.close()
            self.file = None


def _num(v: str):
    try:
        return int(v)
    except ValueError:
        try:
            return float(v)
        except ValueError:
            return v


class ThroughputTimer:
    """Samples/s accumulated over step wall time only (evaluation and checkpoint time excluded
    because the timer is stopped around them), as the reference's ``ThroughputTimer``
    (primus_mllog/mlperf_logger.py:120-156)."""

    def __init__(self, samples_per_step: int, clock: Callable[[], float] = time.perf_counter):
        self.samples_per_step = samples_per_step
        self.clock = clock
        self.total_s = 0.0
        self.steps = 0
        self._t0: float | None = None

    def step_start(self) -> None:
        self._t0 = self.clock()

    def step_stop(self) -> float:
        if self._t0 is None:
            return 0.0
        dt = self.clock() - self._t0
        self.total_s += dt
        self.steps += 1
        self._t0 = None
        return dt

    @property
    def samples(self) -> int:
        return self.steps * self.samples_per_step

    def throughput(self) -> float:
        return self.samples / self.total_s if self.total_s > 0 else 0.0


def parse_log(text: str) -> list[dict]:
    out = []
    for line in text.splitlines():
        i = line.find(PREFIX)
        if i >= 0:
            try:
                out.append(json.loads(line[i + len(PREFIX):].strip()))
            except json.JSONDecodeError:
                pass
    return out


def check_compliance(records: list[dict]) -> list[str]:
    """Structural checks of one trial log (the offline stand-in for
    ``mlperf_logging.compliance_checker --usage training`` that the reference's launcher runs on
    every trial, small_llm_pretraining/primus/run_with_docker.sh:146-152).  Returns problems."""
    problems = []
    keys = [r["key"] for r in records]

    def first(k):
        return keys.index(k) if k in keys else -1

    for k in (INIT_START, INIT_STOP, RUN_START, RUN_STOP, SUBMISSION_BENCHMARK, GLOBAL_BATCH_SIZE):
        if k not in keys:
            problems.append(f"missing {k}")
    order = [CACHE_CLEAR, INIT_START, INIT_STOP, RUN_START, RUN_STOP]
    idx = [first(k) for k in order if k in keys]
    if idx != sorted(idx):
        problems.append("lifecycle events out of order")
    times = [r["time_ms"] for r in records]
    if times != sorted(times):
        problems.append("time stamps decrease")
    if keys.count(RUN_START) > 1 or keys.count(RUN_STOP) > 1:
        problems.append("run_start/run_stop logged more than once")
    depth = 0
    for r in records:
        if r["key"] == BLOCK_START:
            depth += 1
        elif r["key"] == BLOCK_STOP:
            depth -= 1
        if depth < 0 or depth > 1:
            problems.append("block_start/block_stop not paired")
            break
    for r in records:
        if r["key"] == RUN_STOP and r.get("metadata", {}).get("status") not in (SUCCESS, ABORTED):
            problems.append("run_stop without status")
    if EVAL_ACCURACY in keys and first(EVAL_ACCURACY) < first(RUN_START):
        problems.append("eval_accuracy before run_start")
    return problems
