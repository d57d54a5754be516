"""Evaluation cadence expressed as fractions of the training data, turned into global steps.

Pure functions (no torch, no process group), so every rank computes the same thresholds from the
same inputs and no rank can disagree about whether an evaluation boundary is skipped - a
disagreement would leave some ranks inside a collective the others never enter.  Percentages are taken
in sample space against the epoch size and divided once by the global batch size, rounding up, so a
boundary lands at or after the requested fraction.

Reference: generative_recommenders/dlrm_v4/train/utils.py:4140-4226 (``data_pct_to_global_steps``,
``first_data_pct_eval_steps``, ``resolve_skip_eval_until_step`` with the MLPerf first-evaluation rule for
the HSTU benchmark).
"""
from __future__ import annotations

import math


def data_pct_to_global_steps(data_pct: float, total_train_samples: int, global_batch_size: int) -> int:
    """Steps that cover ``data_pct`` (a fraction, 0.01 = 1 %) of the epoch; 0 when any input is not positive."""
    if data_pct <= 0 or total_train_samples <= 0 or global_batch_size <= 0:
        return 0
    return int(math.ceil(data_pct * float(total_train_samples) / float(global_batch_size)))


def skip_eval_until_step(skip_eval_epoch_pct: float, total_train_samples: int, global_batch_size: int) -> int:
    """First global step at which a periodic evaluation may run (boundaries at smaller steps are skipped).
    A negative fraction selects the MLPerf rule: the first evaluation lands at
    ``ceil(floor((4480 GBS + 135331840) / 3) / I) * I`` samples with ``I = ceil(0.001 total / GBS) * GBS``."""
    if skip_eval_epoch_pct < 0:
        if total_train_samples <= 0 or global_batch_size <= 0:
            return 0
        interval = math.ceil(0.001 * float(total_train_samples) / float(global_batch_size)) * global_batch_size
        first = math.floor((4480 * global_batch_size + 135331840) / 3)
        first = int(math.ceil(first / interval)) * interval
        return first // global_batch_size
    return data_pct_to_global_steps(skip_eval_epoch_pct, total_train_samples, global_batch_size)


def first_eval_steps(gstep0: int, eval_interval_steps: int, skip_until_step: int) -> int:
    """Training steps from global step ``gstep0`` to the first evaluation of a loop that evaluates after the
    step that makes the global step ``g`` when ``g > 0``, ``g % eval_interval_steps == 0`` and
    ``g >= skip_until_step``; 0 when the cadence is off."""
    if eval_interval_steps <= 0:
        return 0
    lo = max(int(gstep0) + 1, int(skip_until_step), 1)
    first = -(-lo // int(eval_interval_steps)) * int(eval_interval_steps)
    return first - int(gstep0)


def should_eval(global_step: int, eval_interval_steps: int, skip_until_step: int = 0) -> bool:
    """Whether the loop evaluates after the step that made the global step ``global_step``."""
    return (eval_interval_steps > 0 and global_step > 0 and global_step % eval_interval_steps == 0
            and global_step >= skip_until_step)
