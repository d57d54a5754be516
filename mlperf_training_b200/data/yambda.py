"""Memory-mapped flat event store for the recommender workload (Yambda-style listening events).

Store layout (``write_event_store``): four parallel ``.npy`` arrays sorted by ``(user, timestamp)``
- ``user`` int64, ``item`` int64, ``ts`` int64 (seconds), ``kind`` uint8 (0 listen, 1 like, 2 skip, ...)
plus ``user_offsets`` (CSR over users).  Nothing is loaded eagerly: the arrays are ``np.load(...,
mmap_mode="r")`` views, so a worker touches only the bytes of the samples it builds.

Sampling follows the reference's loader (generative_recommenders/dlrm_v4/datasets/yambda.py:155-246,
668-960, 1415-1657):

* an *anchor* is a listen event with at least ``min_history`` earlier events of the same user; the
  anchor is the target, its label bit is "listened past the threshold" (``kind == 0`` and ``played``);
* the history is the user's events before the anchor, drawn from three pools (listen / like / skip)
  capped at ``max_history // 3`` each, most recent first, then merged back in time order;
* anchors are grouped into windows of ``window_seconds`` (86,400 in the reference); a run walks the
  windows in time order, every rank taking a deterministic slice of each window;
* users are split into train / hold-out by a salted hash of the user id, so a resumed run keeps
  the split as long as the salt and fraction are unchanged (the checkpoint's split contract).

``batch_at`` returns the same dictionary as ``data.hstu_synth.HSTUSyntheticData.batch_at``.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

from .prep import build_window_index


def write_event_store(root: str, user: np.ndarray, item: np.ndarray, ts: np.ndarray, kind: np.ndarray,
                      played: np.ndarray | None = None) -> None:
    order = np.lexsort((ts, user))
    user, item, ts, kind = user[order], item[order], ts[order], kind[order]
    played = np.ones_like(kind) if played is None else played[order]
    d = Path(root)
    d.mkdir(parents=True, exist_ok=True)
    n_users = int(user.max()) + 1 if len(user) else 0
    offsets = np.zeros(n_users + 1, dtype=np.int64)
    np.add.at(offsets, user + 1, 1)
    offsets = np.cumsum(offsets)
    for name, arr in (("user", user.astype(np.int64)), ("item", item.astype(np.int64)), ("ts", ts.astype(np.int64)),
                      ("kind", kind.astype(np.uint8)), ("played", played.astype(np.uint8)), ("user_offsets", offsets)):
        np.save(d / f"{name}.npy", arr)


def convert_sessions(processed_dir: str, metadata_dir: str | None, root: str, listen_plus_threshold: float = 50.0) -> int:
    """The preprocessed public data of the reference -> an event store under ``root``.

    ``processed_dir/train_sessions.parquet`` holds one row per session with list columns ``item_ids``, ``timestamps``,
    ``event_types`` (0 listen, 1 like, others), ``played_ratio_pct`` beside ``uid`` / ``session_id``
    (generative_recommenders/dlrm_v4/datasets/yambda.py:156-212); ``metadata_dir/{artist,album}_item_mapping.parquet`` map an
    ``item_id`` to its ``artist_id`` / ``album_id`` (``:623-636``).  Events keep their type (listens stay anchors whatever
    their played ratio); ``played`` is 1 for a listen played for at least ``listen_plus_threshold`` percent - the
    listen-plus label.  Returns the number of events."""
    import pandas as pd
    df = pd.read_parquet(Path(processed_dir) / "train_sessions.parquet").sort_values(["uid", "session_id"], kind="stable")
    lens = df["item_ids"].map(len).to_numpy()
    user = np.repeat(df["uid"].to_numpy().astype(np.int64), lens)
    flat = lambda c, dt: np.concatenate([np.asarray(v) for v in df[c]]).astype(dt) if len(df) else np.zeros(0, dt)
    item, ts, kind = flat("item_ids", np.int64), flat("timestamps", np.int64), flat("event_types", np.int64)
    ratio = np.nan_to_num(flat("played_ratio_pct", np.float32), nan=0.0)
    played = ((kind == 0) & (ratio >= listen_plus_threshold)).astype(np.uint8)
    write_event_store(root, user, item, ts, kind.clip(0, 255), played)
    if metadata_dir is not None:
        n_items = int(item.max()) + 1 if len(item) else 0
        for name in ("artist", "album"):
            f = Path(metadata_dir) / f"{name}_item_mapping.parquet"
            if f.exists():
                m = pd.read_parquet(f)
                table = np.zeros(max(n_items, int(m["item_id"].max()) + 1), dtype=np.int64)
                table[m["item_id"].to_numpy()] = m[f"{name}_id"].to_numpy()
                np.save(Path(root) / f"item_{name}.npy", table)
    return int(len(user))


def write_synthetic_event_store(root: str, users: int, events_per_user: int, items: int, *, days: int = 7,
                                zipf_alpha: float = 1.05, seed: int = 0) -> int:
    """A random event store for runs without the real data: item popularity follows a bounded Zipf
    law, every user's events are spread over ``days`` days in time order, three in five events are
    listens (four in five of them played through), the rest likes and skips.  Returns the number of
    events.  (The reference ships a generator of synthetic streaming data for the same purpose:
    generative_recommenders/dlrm_v4/streaming_synthetic_data.py.)"""
    rng = np.random.default_rng(seed)
    n = users * events_per_user
    ranks = np.arange(1, items + 1, dtype=np.float64)
    p = ranks ** -zipf_alpha
    item = rng.choice(items, size=n, p=p / p.sum())
    user = np.repeat(np.arange(users), events_per_user)
    ts = 1_600_000_000 + rng.integers(0, days * 86_400, size=n)
    kind = rng.choice(np.array([0, 0, 0, 1, 2], dtype=np.uint8), size=n)
    played = (rng.random(n) < 0.8).astype(np.uint8)
    write_event_store(root, user, item, ts, kind, played)
    return n


def _user_hash(user: np.ndarray, salt: int) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = user.astype(np.uint64) + np.uint64(salt) * np.uint64(0x9E3779B97F4A7C15) + np.uint64(1)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return (z >> np.uint64(40)).astype(np.float64) / float(1 << 24)


class EventStoreDataset:
    def __init__(self, root: str, batch: int, *, max_history: int = 4086, min_history: int = 16,
                 window_seconds: int = 86_400, holdout: float = 0.05, salt: int = 0, split: str = "train"):
        d = Path(root)
        self.user, self.item, self.ts, self.kind, self.played, self.uoff = (
            np.load(d / f"{n}.npy", mmap_mode="r") for n in ("user", "item", "ts", "kind", "played", "user_offsets"))
        self.batch, self.max_history, self.min_history = batch, max_history, min_history
        self.num_items = int(np.asarray(self.item).max()) + 1 if len(self.item) else 0     # the table must have this many rows
        # optional item -> artist / album maps (``item_artist.npy`` / ``item_album.npy``, indexed by item id) for the
        # multi-table feature set; without them the features fall back to an arithmetic map of the item id
        self.item_artist = torch.from_numpy(np.load(d / "item_artist.npy").astype(np.int64)) if (d / "item_artist.npy").exists() else None
        self.item_album = torch.from_numpy(np.load(d / "item_album.npy").astype(np.int64)) if (d / "item_album.npy").exists() else None
        self.contract = {"window_seconds": window_seconds, "holdout": holdout, "salt": salt}
        # anchors: listen events with enough history, of users on this side of the split
        pos_in_user = np.arange(len(self.user)) - np.asarray(self.uoff)[np.asarray(self.user)]
        is_anchor = (np.asarray(self.kind) == 0) & (pos_in_user >= min_history)
        held = _user_hash(np.asarray(self.user), salt) < holdout
        keep = is_anchor & (held if split == "eval" else ~held)
        self.anchors = np.flatnonzero(keep)
        idx = build_window_index(np.asarray(self.ts)[self.anchors], window_seconds)
        self.order, self.window_start = idx["order"], np.r_[idx["window_start"], len(self.anchors)]

    # ------------------------------------------------------------------ windows
    @property
    def num_windows(self) -> int:
        return len(self.window_start) - 1

    def window_anchors(self, w: int, rank: int = 0, world: int = 1) -> np.ndarray:
        """This rank's anchors of window ``w`` in time order (every ``world``-th anchor)."""
        ids = self.anchors[self.order[self.window_start[w]:self.window_start[w + 1]]]
        return ids[rank::world]

    def batches_in_window(self, w: int, world: int = 1) -> int:
        n = self.window_start[w + 1] - self.window_start[w]
        return int(n // (world * self.batch))            # every rank runs the same number of steps

    # ------------------------------------------------------------------ samples
    def _history(self, anchor: int) -> np.ndarray:
        u = int(self.user[anchor])
        lo = int(self.uoff[u])
        ev = np.arange(lo, anchor)
        kinds = np.asarray(self.kind[lo:anchor])
        cap = self.max_history // 3
        picked = [ev[kinds == k][-cap:] for k in (0, 1, 2)]
        rest = ev[kinds > 2][-max(self.max_history - sum(len(p) for p in picked), 0):]
        return np.sort(np.concatenate(picked + [rest]))

    def build_batch(self, anchors: np.ndarray, pin: bool = False) -> dict:
        hists = [self._history(int(a)) for a in anchors]
        lens = np.array([len(h) + 1 for h in hists], dtype=np.int64)
        offsets = np.zeros(len(anchors) + 1, dtype=np.int32)
        offsets[1:] = np.cumsum(lens)
        total = int(offsets[-1])
        ev = np.concatenate([np.r_[h, a] for h, a in zip(hists, anchors)])
        ids = np.asarray(self.item)[ev]
        ts = np.asarray(self.ts)[ev]
        kind = np.asarray(self.kind)[ev].astype(np.int64)
        played = np.asarray(self.played)[ev].astype(np.int64)
        actions = (((kind == 0) & (played > 0)).astype(np.int64) | ((kind == 1).astype(np.int64) << 1)
                   | ((kind == 2).astype(np.int64) << 2))
        out = {"offsets": torch.from_numpy(offsets), "num_targets": torch.ones(len(anchors), dtype=torch.int32),
               "timestamps": torch.from_numpy(ts.astype(np.int64)), "actions": torch.from_numpy(actions),
               "item_ids": torch.from_numpy(ids.astype(np.int64)), "total": total, "rows": (total + 127) // 128 * 128,
               "lengths": torch.from_numpy(lens), "max_targets": 1,
               "users": torch.from_numpy(np.asarray(self.user)[anchors].astype(np.int64))}
        if pin and torch.cuda.is_available():
            out = {k: (v.pin_memory() if torch.is_tensor(v) else v) for k, v in out.items()}
        return out

    def batch_in_window(self, w: int, k: int, rank: int = 0, world: int = 1, pin: bool = False) -> dict:
        ids = self.window_anchors(w, rank, world)
        return self.build_batch(ids[k * self.batch:(k + 1) * self.batch], pin)

    # ------------------------------------------------------------------ read-ahead
    def step_anchors(self, step: int, rank: int = 0, world: int = 1) -> np.ndarray:
        """Anchor events of this rank's batch at stream step ``step``."""
        w = self.window_of_step(step, world)
        k = step % max(sum(self.batches_in_window(x, world) for x in range(self.num_windows)), 1)
        k -= sum(self.batches_in_window(x, world) for x in range(w))
        return self.window_anchors(w, rank, world)[k * self.batch:(k + 1) * self.batch]

    def event_ranges(self, steps, rank: int = 0, world: int = 1) -> list[tuple[int, int]]:
        """Merged ``[lo, hi)`` event-index ranges that the batches of ``steps`` read: for every anchor its
        user's events from the first one up to the anchor itself."""
        spans = []
        for s in steps:
            for a in self.step_anchors(int(s), rank, world):
                spans.append((int(self.uoff[int(self.user[a])]), int(a) + 1))
        spans.sort()
        merged: list[list[int]] = []
        for lo, hi in spans:
            if merged and lo <= merged[-1][1]:
                merged[-1][1] = max(merged[-1][1], hi)
            else:
                merged.append([lo, hi])
        return [(lo, hi) for lo, hi in merged]

    def prefetch(self, steps, rank: int = 0, world: int = 1) -> int:
        """Ask the kernel to read ahead (``posix_fadvise(WILLNEED)``) exactly the bytes of the per-event
        arrays that the batches of ``steps`` will touch, so a cold page cache is filled while earlier steps
        run instead of stalling the loader (generative_recommenders/dlrm_v4/train/cold_prefetch.py).  Returns
        the number of bytes advised; 0 where the call is not available."""
        import os
        if not hasattr(os, "posix_fadvise"):
            return 0
        ranges, total = self.event_ranges(steps, rank, world), 0
        for arr in (self.item, self.ts, self.kind, self.played):
            name, base, width = getattr(arr, "filename", None), int(getattr(arr, "offset", 0)), arr.dtype.itemsize
            if name is None:
                continue
            fd = os.open(name, os.O_RDONLY)
            try:
                for lo, hi in ranges:
                    os.posix_fadvise(fd, base + lo * width, (hi - lo) * width, os.POSIX_FADV_WILLNEED)
                    total += (hi - lo) * width
            finally:
                os.close(fd)
        return total

    def window_of_step(self, step: int, world: int = 1) -> int:
        """Index of the time window that step ``step`` of the stream reads from."""
        per_window = [self.batches_in_window(w, world) for w in range(self.num_windows)]
        total = sum(per_window)
        if total == 0:
            raise IndexError("no window holds a full batch for every rank")
        step %= total
        for w, n in enumerate(per_window):
            if step < n:
                return w
            step -= n
        return self.num_windows - 1

    def batch_at(self, step: int, rank: int = 0, pin: bool = False, world: int = 1) -> dict:
        """Step ``step`` of the stream that walks the windows in order (exact-once: a resumed run that
        asks for the same step gets the same samples)."""
        per_window = [self.batches_in_window(w, world) for w in range(self.num_windows)]
        total = sum(per_window)
        if total == 0:
            raise IndexError("no window holds a full batch for every rank")
        step %= total                                   # a further pass over the stream starts at the first window
        for w, n in enumerate(per_window):
            if step < n:
                return self.batch_in_window(w, step, rank, world, pin)
            step -= n
