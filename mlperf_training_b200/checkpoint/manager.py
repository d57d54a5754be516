"""Crash-safe checkpoint directories and exact resume bookkeeping.

Layout ``<root>/<N>/`` where ``N`` is the global step (or window id):

    dense.pt            model (non-sharded) state, scheduler position, run markers   (rank 0)
    optim_rank<r>.pt    this rank's shard of the optimizer state
    rng_rank<r>.pt      per-rank RNG streams (CPU + CUDA)
    sparse/             sharded embedding tables (one file per rank + metadata), optional
    meta.json           step, samples consumed, position inside the data window, split contract

Protocol (all ranks call ``save``; the callable ``barrier`` keeps them in step):
rank 0 sweeps stale ``*.tmp`` and creates ``<N>.tmp`` -> barrier -> every rank writes its files ->
barrier -> rank 0 renames ``<N>.tmp`` to ``<N>`` (moving an existing ``<N>`` aside first) and prunes to
``keep_last`` -> barrier.  A directory without the ``.tmp`` suffix is therefore always complete.

Same protocol and cadence rules as the reference's recommender checkpointing
(generative_recommenders/dlrm_v4/checkpoint.py:338-525 save, :527-716 load;
generative_recommenders/dlrm_v4/train/utils.py:4097-4226 cadence decisions).
"""
from __future__ import annotations

import json
import os
import shutil
import time
from pathlib import Path
from typing import Callable

import torch

WINDOW_COMPLETE = -1


def _noop() -> None:
    return None


class CheckpointManager:
    def __init__(self, root: str, rank: int = 0, world: int = 1, keep_last: int = 2,
                 barrier: Callable[[], None] | None = None):
        self.root = Path(root)
        self.rank, self.world, self.keep_last = rank, world, keep_last
        self.barrier = barrier or _noop

    # ------------------------------------------------------------------ discovery
    def steps(self) -> list[int]:
        if not self.root.exists():
            return []
        return sorted(int(p.name) for p in self.root.iterdir() if p.is_dir() and p.name.isdigit())

    def latest(self) -> int | None:
        s = self.steps()
        return s[-1] if s else None

    def present(self) -> bool:
        return self.latest() is not None

    def path(self, step: int) -> Path:
        return self.root / str(step)

    # ------------------------------------------------------------------ save
    def save(self, step: int, *, dense: dict | None, optim_shard: dict | None, meta: dict,
             sparse_writer: Callable[[Path], None] | None = None, save_rng: bool = True) -> Path:
        tmp = self.root / f"{step}.tmp"
        final = self.path(step)
        if self.rank == 0:
            self.root.mkdir(parents=True, exist_ok=True)
            for stale in self.root.glob("*.tmp"):
                shutil.rmtree(stale, ignore_errors=True)
            (tmp / "sparse").mkdir(parents=True, exist_ok=True)
        self.barrier()
        if self.rank == 0 and dense is not None:
            torch.save(dense, tmp / "dense.pt")
        if optim_shard is not None:
            torch.save(optim_shard, tmp / f"optim_rank{self.rank}.pt")
        if save_rng:
            rng = {"cpu": torch.get_rng_state()}
            if torch.cuda.is_available():
                rng["cuda"] = torch.cuda.get_rng_state()
            torch.save(rng, tmp / f"rng_rank{self.rank}.pt")
        if sparse_writer is not None:
            sparse_writer(tmp / "sparse")
        if self.rank == 0:
            meta = dict(meta, step=step, world=self.world, saved_at=time.time())
            (tmp / "meta.json").write_text(json.dumps(meta, indent=1))
        self.barrier()
        if self.rank == 0:
            if final.exists():
                aside = self.root / f"{step}.old.tmp"
                shutil.rmtree(aside, ignore_errors=True)
                os.rename(final, aside)
            os.rename(tmp, final)
            shutil.rmtree(self.root / f"{step}.old.tmp", ignore_errors=True)
            (self.root / "latest_checkpointed_iteration.txt").write_text(str(step))
            for old in self.steps()[:-self.keep_last] if self.keep_last > 0 else []:
                shutil.rmtree(self.path(old), ignore_errors=True)
        self.barrier()
        return final

    # ------------------------------------------------------------------ asynchronous save
    def save_async(self, step: int, *, dense: dict | None, optim_shard: dict | None, meta: dict, save_rng: bool = True):
        """Snapshot the tensors to host memory now and write the checkpoint on a background thread, so
        the training loop only pays for the device-to-host copy.  ``finalize_async()`` must be called
        (it is called by the next ``save`` / ``save_async`` too) before the checkpoint counts as
        complete - the async save + finalisation hook of the reference's SFT loop
        (llama2_sft/primus/src/llama2_custom.py:1859-1863).  Single-process writers only: the barriers
        of ``save`` cannot run on a side thread, so with ``world > 1`` this falls back to ``save``."""
        import threading
        self.finalize_async()
        if self.world > 1:
            return self.save(step, dense=dense, optim_shard=optim_shard, meta=meta, save_rng=save_rng)

        def to_host(obj):
            if torch.is_tensor(obj):
                return obj.detach().to("cpu", copy=True)
            if isinstance(obj, dict):
                return {k: to_host(v) for k, v in obj.items()}
            if isinstance(obj, (list, tuple)):
                return type(obj)(to_host(v) for v in obj)
            return obj
        dense_h, optim_h = to_host(dense), to_host(optim_shard)
        rng = None
        if save_rng:
            rng = {"cpu": torch.get_rng_state()}
            if torch.cuda.is_available():
                rng["cuda"] = torch.cuda.get_rng_state()
        result: dict = {}

        def work():
            try:
                result["path"] = self._write(step, dense_h, optim_h, meta, rng)
            except Exception as e:      # surfaced by finalize_async
                result["error"] = e
        t = threading.Thread(target=work, name="checkpoint-writer", daemon=True)
        t.start()
        self._pending = (t, result)
        return None

    def finalize_async(self):
        """Wait for the background write; returns its path (None when nothing was pending)."""
        pending = getattr(self, "_pending", None)
        if pending is None:
            return None
        t, result = pending
        t.join()
        self._pending = None
        if "error" in result:
            raise result["error"]
        return result.get("path")

    def _write(self, step: int, dense, optim_shard, meta: dict, rng) -> Path:
        tmp, final = self.root / f"{step}.tmp", self.path(step)
        self.root.mkdir(parents=True, exist_ok=True)
        shutil.rmtree(tmp, ignore_errors=True)
        (tmp / "sparse").mkdir(parents=True, exist_ok=True)
        if dense is not None:
            torch.save(dense, tmp / "dense.pt")
        if optim_shard is not None:
            torch.save(optim_shard, tmp / f"optim_rank{self.rank}.pt")
        if rng is not None:
            torch.save(rng, tmp / f"rng_rank{self.rank}.pt")
        (tmp / "meta.json").write_text(json.dumps(dict(meta, step=step, world=self.world, saved_at=time.time()), indent=1))
        if final.exists():
            shutil.rmtree(final, ignore_errors=True)
        os.rename(tmp, final)
        (self.root / "latest_checkpointed_iteration.txt").write_text(str(step))
        for old in self.steps()[:-self.keep_last] if self.keep_last > 0 else []:
            shutil.rmtree(self.path(old), ignore_errors=True)
        return final

    # ------------------------------------------------------------------ load
    def load(self, step: int | None = None, map_location="cpu") -> dict | None:
        """Returns ``{"dense", "optim", "rng", "meta", "path"}`` of ``step`` (default: latest
        complete one) or None when there is no checkpoint."""
        step = self.latest() if step is None else step
        if step is None:
            return None
        d = self.path(step)
        out = {"path": d, "meta": json.loads((d / "meta.json").read_text())}
        out["dense"] = torch.load(d / "dense.pt", map_location=map_location, weights_only=False) if (d / "dense.pt").exists() else None
        f = d / f"optim_rank{self.rank}.pt"
        out["optim"] = torch.load(f, map_location=map_location, weights_only=False) if f.exists() else None
        f = d / f"rng_rank{self.rank}.pt"
        out["rng"] = torch.load(f, map_location="cpu", weights_only=False) if f.exists() else None
        return out

    @staticmethod
    def restore_rng(rng: dict | None) -> None:
        if not rng:
            return
        torch.set_rng_state(rng["cpu"])
        if "cuda" in rng and torch.cuda.is_available():
            torch.cuda.set_rng_state(rng["cuda"])


# --------------------------------------------------------------------------------------
# pure cadence / resume decisions (torch-free, unit-testable)
# --------------------------------------------------------------------------------------
def select_checkpoint_reason(*, global_step: int, batch_in_window: int, elapsed_since_last_s: float,
                             every_steps: int = 0, every_window_batches: int = 0, every_seconds: float = 0.0,
                             window_end: bool = False, at_window_end: bool = True) -> str | None:
    """Why a checkpoint is due now, or None.  Priority: window end, step cadence, in-window batch
    cadence, wall clock (``elapsed_since_last_s`` is rank 0's clock, broadcast by the caller)."""
    if window_end and at_window_end:
        return "window"
    if every_steps > 0 and global_step > 0 and global_step % every_steps == 0:
        return "global_step"
    if every_window_batches > 0 and batch_in_window > 0 and batch_in_window % every_window_batches == 0:
        return "in_window"
    if every_seconds > 0 and elapsed_since_last_s >= every_seconds:
        return "wall_clock"
    return None


def resume_position(meta: dict | None, batch_size_per_rank: int) -> dict:
    """Where to continue: ``window`` to enter, ``skip_batches`` / ``skip_samples`` of this rank's
    deterministic slice of that window already consumed.  ``batch_idx_in_window ==
    WINDOW_COMPLETE`` means the saved window finished: start the next one from its beginning."""
    if not meta:
        return {"window": 0, "skip_batches": 0, "skip_samples": 0, "cold_start": True}
    w = int(meta.get("window", 0))
    k = int(meta.get("batch_idx_in_window", WINDOW_COMPLETE))
    if k == WINDOW_COMPLETE:
        return {"window": w + 1, "skip_batches": 0, "skip_samples": 0, "cold_start": False}
    return {"window": w, "skip_batches": k, "skip_samples": k * batch_size_per_rank, "cold_start": False}


def validate_split_contract(saved: dict | None, current: dict, allow_mismatch: bool = False) -> None:
    """The train/eval split parameters of a resumed run must equal those of the run that wrote the
    checkpoint (salt, holdout fraction, window length, world size) unless explicitly allowed."""
    if saved is None or allow_mismatch:
        return
    bad = {k: (saved.get(k), current.get(k)) for k in current if saved.get(k) != current.get(k)}
    if bad:
        raise RuntimeError(f"checkpoint split contract mismatch: {bad}")
