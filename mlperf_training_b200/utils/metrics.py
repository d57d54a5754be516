"""Recommender evaluation metrics: exact (sort-based) window AUC, additive binned cumulative AUC,
normalised entropy and accuracy.

``window_auc`` is the target metric of the recommender workload (``EVAL_ACCURACY`` = window AUC of
the holdout pass, compared against ``AUC_THRESHOLD`` = 0.75;
generative_recommenders/dlrm_v4/train/mlperf_logging_utils.py:671,731-745,803-826): predictions of
all ranks are gathered and ranked.  ``BinnedCumulativeAUC`` keeps two float64 histograms of
positive / negative weight over ``bins`` score bins; its state is additive, so cross-rank
synchronisation is a sum all-reduce and it can be checkpointed
(generative_recommenders/dlrm_v4/utils.py:188-280).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def exact_auc(scores: torch.Tensor, labels: torch.Tensor, weights: torch.Tensor | None = None) -> float:
    """Weighted ROC AUC with ties counted half (0.5 when one class is absent)."""
    s = scores.double().reshape(-1)
    y = labels.double().reshape(-1)
    w = torch.ones_like(s) if weights is None else weights.double().reshape(-1)
    pos_w, neg_w = (w * y).sum(), (w * (1 - y)).sum()
    if pos_w <= 0 or neg_w <= 0:
        return 0.5
    order = torch.argsort(s, stable=True)
    s, y, w = s[order], y[order], w[order]
    # group ties
    new = torch.ones_like(s, dtype=torch.bool)
    new[1:] = s[1:] != s[:-1]
    gid = torch.cumsum(new.long(), 0) - 1
    n = int(gid[-1]) + 1
    pos_g = torch.zeros(n, dtype=torch.float64, device=s.device).index_add_(0, gid, w * y)
    neg_g = torch.zeros(n, dtype=torch.float64, device=s.device).index_add_(0, gid, w * (1 - y))
    neg_below = torch.cumsum(neg_g, 0) - neg_g
    return float((pos_g * (neg_below + 0.5 * neg_g)).sum() / (pos_w * neg_w))


def gather_all(t: torch.Tensor) -> torch.Tensor:
    """Concatenate variable-length 1-D tensors of all ranks."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return t
    n = torch.tensor([t.numel()], dtype=torch.int64, device=t.device)
    sizes = [torch.zeros_like(n) for _ in range(dist.get_world_size())]
    dist.all_gather(sizes, n)
    m = int(max(int(s) for s in sizes))
    pad = torch.zeros(m, dtype=t.dtype, device=t.device)
    pad[: t.numel()] = t
    bufs = [torch.zeros_like(pad) for _ in sizes]
    dist.all_gather(bufs, pad)
    return torch.cat([b[: int(s)] for b, s in zip(bufs, sizes)])


def window_auc(scores: torch.Tensor, labels: torch.Tensor, weights: torch.Tensor | None = None) -> float:
    s, y = gather_all(scores.float()), gather_all(labels.float())
    w = None if weights is None else gather_all(weights.float())
    return exact_auc(s, y, w)


class BinnedCumulativeAUC:
    def __init__(self, n_tasks: int = 1, bins: int = 100_000, device="cpu"):
        self.bins = bins
        self.pos = torch.zeros(n_tasks, bins, dtype=torch.float64, device=device)
        self.neg = torch.zeros(n_tasks, bins, dtype=torch.float64, device=device)

    def update(self, scores: torch.Tensor, labels: torch.Tensor, weights: torch.Tensor | None = None, task: int = 0):
        b = (scores.double() * self.bins).long().clamp(0, self.bins - 1)
        w = torch.ones_like(scores, dtype=torch.float64) if weights is None else weights.double()
        y = labels.double()
        self.pos[task].index_add_(0, b, w * y)
        self.neg[task].index_add_(0, b, w * (1 - y))

    def sync(self) -> None:
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(self.pos)
            dist.all_reduce(self.neg)

    def compute(self, task: int = 0) -> float:
        pos, neg = self.pos[task], self.neg[task]
        denom = pos.sum() * neg.sum()
        if denom <= 0:
            return 0.5
        neg_below = torch.cumsum(neg, 0) - neg
        return float((pos * (neg_below + 0.5 * neg)).sum() / denom)

    def state_dict(self):
        return {"pos": self.pos, "neg": self.neg}

    def load_state_dict(self, sd):
        self.pos.copy_(sd["pos"])
        self.neg.copy_(sd["neg"])


def grouped_auc(scores: torch.Tensor, labels: torch.Tensor, groups: torch.Tensor) -> float:
    """GAUC: the AUC computed inside each group (user) and averaged with the group's sample count as
    weight; groups with a single class are skipped (the per-user AUC the reference's metrics logger
    reports next to the global one, generative_recommenders/dlrm_v4/utils.py:842-1535)."""
    tot, wsum = 0.0, 0.0
    for g in torch.unique(groups):
        m = groups == g
        y = labels[m]
        if y.min() == y.max():
            continue
        n = int(m.sum())
        tot += n * exact_auc(scores[m], y)
        wsum += n
    return tot / wsum if wsum > 0 else 0.5


def normalized_entropy(scores: torch.Tensor, labels: torch.Tensor, eps: float = 1e-12) -> float:
    p = scores.double().clamp(eps, 1 - eps)
    y = labels.double()
    ce = -(y * p.log() + (1 - y) * (1 - p).log()).mean()
    base = y.mean().clamp(eps, 1 - eps)
    return float(ce / -(base * base.log() + (1 - base) * (1 - base).log()))


def accuracy(scores: torch.Tensor, labels: torch.Tensor, threshold: float = 0.5) -> float:
    return float(((scores >= threshold).float() == labels.float()).float().mean())


class PerfLogger:
    """Per-interval performance line: samples/s, step time, algorithmic TFLOP/s per GPU and MFU, with
    checkpoint / evaluation time excluded through ``pause`` (the reference's ``MetricsLogger`` perf
    line, generative_recommenders/dlrm_v4/utils.py:842-1535), and a durable ``metrics.jsonl``."""

    def __init__(self, flops_per_sample: float, world: int = 1, peak_tflops: float = 2250.0, jsonl: str | None = None):
        import time
        self._now = time.perf_counter
        self.flops_per_sample, self.world, self.peak = flops_per_sample, world, peak_tflops
        self.jsonl = jsonl
        self.t0 = self._now()
        self.paused = 0.0
        self._pause_t = None
        self.samples = 0
        self.steps = 0

    def pause(self) -> None:
        self._pause_t = self._now()

    def resume(self) -> None:
        if self._pause_t is not None:
            self.paused += self._now() - self._pause_t
            self._pause_t = None

    def step(self, samples: int) -> None:
        self.samples += samples
        self.steps += 1

    def line(self, step: int, extra: dict | None = None) -> dict:
        import json
        dt = max(self._now() - self.t0 - self.paused, 1e-9)
        sps = self.samples / dt
        tflops_gpu = sps * self.flops_per_sample / self.world / 1e12
        rec = {"step": step, "samples_per_s": sps, "step_ms": 1e3 * dt / max(self.steps, 1), "tflops_algo_per_gpu": tflops_gpu,
               "mfu": (tflops_gpu / self.peak) if self.peak > 0 else 0.0, **(extra or {})}
        if self.jsonl:
            with open(self.jsonl, "a") as f:
                f.write(json.dumps(rec) + "\n")
        self.t0, self.paused, self.samples, self.steps = self._now(), 0.0, 0, 0
        return rec


def model_fingerprint(model, group=None) -> tuple[str, list[tuple[str, float, float, float]]]:
    """Whole-model initialisation fingerprint: for every parameter in name order the element count,
    the sum and the sum of squares in fp64, and a SHA-256 over those numbers (printed with
    ``INIT_CHECKSUM=1``; two runs that start from the same weights print the same digest).  Parameters
    marked as sharded over ranks (``expert_parallel`` / ``tensor_parallel`` attributes) are summed over
    ``group`` first, so the digest does not depend on which rank prints it
    (generative_recommenders/dlrm_v4/train/utils.py:1695-1748)."""
    import hashlib

    import torch
    import torch.distributed as dist
    rows = []
    for name, p in sorted(model.named_parameters(), key=lambda kv: kv[0]):
        d = p.detach()
        stat = torch.tensor([float(d.numel()), float(d.sum(dtype=torch.float64)), float((d.double() ** 2).sum())],
                            dtype=torch.float64, device=d.device)
        sharded = getattr(p, "expert_parallel", False) or getattr(p, "tensor_parallel", None) is not None
        if sharded and dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(stat, group=group)
        rows.append((name, float(stat[0]), float(stat[1]), float(stat[2])))
    h = hashlib.sha256()
    for name, n, s, q in rows:
        h.update(f"{name}:{n:.0f}:{s:.10e}:{q:.10e};".encode())
    return h.hexdigest(), rows


class StartupTimeline:
    """Named phases of the time before the clock starts (model build, sharding, loaders, checkpoint
    load, warm-ups), each stamped when it ends; ``report()`` gives seconds per phase and the total, which a
    run prints once so that slow cold starts can be told apart from slow steps
    (generative_recommenders/dlrm_v4/train/dl_prestart.py keeps the same kind of startup timeline)."""

    def __init__(self, clock=None):
        import time
        self._clock = clock or time.perf_counter
        self._t0 = self._last = self._clock()
        self.phases: list[tuple[str, float]] = []

    def mark(self, name: str) -> float:
        now = self._clock()
        self.phases.append((name, now - self._last))
        self._last = now
        return self.phases[-1][1]

    def report(self) -> dict:
        return {"phases": {n: round(t, 4) for n, t in self.phases}, "total_s": round(self._last - self._t0, 4)}
