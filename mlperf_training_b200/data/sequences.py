"""Per-user sequence files (MovieLens / KuaiRand style) as HSTU training batches.

A file has one row per user whose cells hold whole sequences, either comma-separated or as JSON
lists: item ids, a per-event signal (ratings for MovieLens, ready-made action bit masks for
KuaiRand) and timestamps.  The last ``num_candidates`` events of a user are the ranking candidates
(targets), everything before them the interaction history; users with no history left are skipped;
a history longer than ``max_history`` keeps its first ``max_history`` events; candidates carry the
query time (the latest history timestamp) instead of their own.  History events get the action
mask ``action_weights[rating - 1]`` (MovieLens) or the stored mask (KuaiRand); a candidate's label
is ``rating >= 3.5`` (MovieLens) or ``mask & label_bit`` (KuaiRand), stored in ``label_bit`` of
its action word, which the model reads as the target and hides from the action encoder.

Batches have the layout of the other HSTU sources (``data/hstu_synth.py``, ``data/yambda.py``): jagged
``item_ids`` / ``timestamps`` / ``actions`` with ``offsets``, ``num_targets`` and the host-known
``total`` / ``rows``.  Users are shuffled per pass with a seed, every rank takes its slice of a step's
users, and the user-hash hold-out of ``data/yambda.py`` gives the train / eval split.

Reference behaviour: generative_recommenders/dlrm_v4/datasets/movie_lens.py:66-177 (history /
candidate split, truncation, query time, rating -> action weight, label >= 3.5),
kuairand.py:51-160 (video_id / action_weights / time_ms columns), datasets/utils.py:41-105 (sequence
parsing, ``separate_uih_candidates``, ``maybe_truncate_seq``), synthetic_movie_lens.py (synthetic files).
"""
from __future__ import annotations

import csv
import json

import numpy as np
import torch

PRESETS = {
    # column names: items, signal, timestamps; whether the signal is a rating (else an action mask)
    "movielens": ("sequence_item_ids", "sequence_ratings", "sequence_timestamps", True),
    "kuairand": ("video_id", "action_weights", "time_ms", False),
}


def parse_sequence(cell) -> list:
    """``"3,5,9"``, ``"[3, 5, 9]"``, ``7`` or a list -> list of numbers."""
    if isinstance(cell, (list, tuple, np.ndarray)):
        return list(cell)
    if isinstance(cell, (int, float)):
        return [cell]
    text = str(cell).strip()
    if not text:
        return []
    if not (text[0] == "[" and text[-1] == "]"):
        text = "[" + text + "]"
    out = json.loads(text)
    return out if isinstance(out, list) else [out]


def split_history_candidates(seq: list, num_candidates: int) -> tuple[list, list]:
    """(history, candidates): the last ``num_candidates`` entries are the candidates."""
    return seq[:-num_candidates], seq[-num_candidates:]


def write_synthetic_sequences(path: str, users: int, items: int, *, min_len: int = 8, max_len: int = 64, seed: int = 0,
                              kind: str = "movielens") -> None:
    """A random file in the layout of ``kind``: lengths uniform in [min_len, max_len], ratings in
    {1, 1.5, ..., 5} (or action masks in [0, 8)), increasing timestamps."""
    rng = np.random.default_rng(seed)
    items_c, signal_c, ts_c, rating = PRESETS[kind]
    with open(path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["user_id", items_c, signal_c, ts_c])
        for u in range(users):
            n = int(rng.integers(min_len, max_len + 1))
            ids = rng.integers(1, items, n)
            sig = rng.integers(2, 11, n) / 2.0 if rating else rng.integers(0, 8, n)
            ts = np.cumsum(rng.integers(1, 10_000, n)) + 1_000_000_000
            w.writerow([u, ",".join(map(str, ids)), ",".join(str(x) for x in sig), ",".join(map(str, ts))])


class SequenceFileDataset:
    def __init__(self, path: str, batch: int, *, kind: str = "movielens", num_candidates: int = 1, max_history: int = 4086,
                 action_weights: tuple = (1, 1, 2, 4, 4), label_bit: int = 1, split: str = "all", eval_fraction: float = 0.1,
                 salt: int = 17, seed: int = 0):
        if kind not in PRESETS:
            raise ValueError(f"unknown sequence file kind '{kind}' (known: {sorted(PRESETS)})")
        items_c, signal_c, ts_c, self.rating = PRESETS[kind]
        self.batch, self.nc, self.max_history, self.seed = batch, int(num_candidates), int(max_history), seed
        self.action_weights, self.label_bit = tuple(action_weights), int(label_bit)
        ids, acts, tss, lens, users = [], [], [], [], []
        with open(path, newline="") as f:
            for n_row, row in enumerate(csv.DictReader(f)):
                for c in (items_c, signal_c, ts_c):
                    if c not in row:
                        raise KeyError(f"{path}: column '{c}' missing (found {sorted(row)})")
                item = parse_sequence(row[items_c])
                if len(item) <= self.nc:
                    continue                                    # nothing left for the history
                sample = self._sample(item, parse_sequence(row[signal_c]), parse_sequence(row[ts_c]))
                ids.append(sample[0]); acts.append(sample[1]); tss.append(sample[2]); lens.append(len(sample[0]))
                users.append(int(row.get("user_id", n_row) or n_row))
        from .yambda import _user_hash
        users = np.asarray(users, dtype=np.int64)
        held = _user_hash(users, salt) < eval_fraction if len(users) else np.zeros(0, bool)
        keep = {"all": np.ones(len(users), bool), "train": ~held, "eval": held}[split]
        self._ids = [a for a, k in zip(ids, keep) if k]
        self._acts = [a for a, k in zip(acts, keep) if k]
        self._ts = [a for a, k in zip(tss, keep) if k]
        self.lengths = np.asarray([n for n, k in zip(lens, keep) if k], dtype=np.int64)

    def __len__(self) -> int:
        return len(self._ids)

    def _sample(self, item: list, signal: list, ts: list):
        if not (len(item) == len(signal) == len(ts)):
            raise ValueError("item, signal and timestamp sequences of a user differ in length")
        (h_i, c_i), (h_s, c_s), (h_t, _) = (split_history_candidates(s, self.nc) for s in (item, signal, ts))
        h_i, h_s, h_t = h_i[:self.max_history], h_s[:self.max_history], h_t[:self.max_history]
        if self.rating:
            h_a = [self.action_weights[int(r) - 1] for r in h_s]
            c_a = [self.label_bit if float(r) >= 3.5 else 0 for r in c_s]
        else:
            h_a = [int(a) for a in h_s]
            c_a = [int(a) & self.label_bit for a in c_s]
        query_time = max(h_t) if h_t else 0
        return (np.asarray(h_i + c_i, dtype=np.int64), np.asarray(h_a + c_a, dtype=np.int64),
                np.asarray(list(h_t) + [query_time] * len(c_i), dtype=np.int64))

    def steps_per_pass(self, world: int = 1) -> int:
        return len(self) // (self.batch * world)

    def build_batch(self, users: np.ndarray, pin: bool = False) -> dict:
        lens = self.lengths[users]
        offsets = np.zeros(len(users) + 1, dtype=np.int32)
        offsets[1:] = np.cumsum(lens)
        total = int(offsets[-1])
        cat = lambda seqs: torch.from_numpy(np.concatenate([seqs[u] for u in users]))       # noqa: E731
        out = {"offsets": torch.from_numpy(offsets), "num_targets": torch.full((len(users),), self.nc, dtype=torch.int32),
               "timestamps": cat(self._ts), "actions": cat(self._acts), "item_ids": cat(self._ids), "total": total,
               "rows": (total + 127) // 128 * 128, "lengths": torch.from_numpy(lens.copy())}
        if pin and torch.cuda.is_available():
            out = {k: (v.pin_memory() if torch.is_tensor(v) else v) for k, v in out.items()}
        return out

    def batch_at(self, step: int, rank: int = 0, pin: bool = False, world: int = 1) -> dict:
        """Users of step ``step`` for ``rank``: pass ``step // steps_per_pass`` shuffles the users with
        its own seed, a step takes ``batch * world`` consecutive users of that order, a rank its slice."""
        per = self.steps_per_pass(world)
        if per == 0:
            raise IndexError(f"{len(self)} users do not fill one step of {self.batch} x {world}")
        order = np.random.default_rng([self.seed, step // per]).permutation(len(self))
        k = (step % per) * self.batch * world + rank * self.batch
        return self.build_batch(order[k:k + self.batch], pin)
