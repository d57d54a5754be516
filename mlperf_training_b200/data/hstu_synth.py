"""Synthetic jagged interaction batches for the HSTU workload.

Per user: a history whose length is log-normal (median ``length_median``) clipped to
``[length_min, length_max]``, followed by one target; item ids Zipf(``zipf_alpha``) over the table;
increasing timestamps; action bit masks.  The target's positive label depends on the item id so a
model can learn it (AUC above chance) - used by the convergence tests.  Stands in for the
reference's synthetic / Yambda loaders (generative_recommenders/dlrm_v4/datasets/dataset.py:1033-1209
``DLRMv4RandomDataset``, yambda.py) with the same batch structure: jagged values + lengths, one
storage per batch, pinned for the H2D copy.

``balance_world = W > 1``: the lengths of a step's W x batch users are drawn once, identically on every rank, and
dealt to the ranks longest first, each to the least loaded rank with a free slot, so every rank gets the same number of
users and nearly the same attention work (which goes with the sum of squared lengths).  The global batch is the same set of i.i.d.
users either way; only their placement changes, and with it the time the slowest rank takes.
"""
from __future__ import annotations

import numpy as np
import torch


class HSTUSyntheticData:
    def __init__(self, rows: int, batch: int, length_median: int = 512, length_min: int = 16, length_max: int = 4096,
                 zipf_alpha: float = 1.05, sigma: float = 1.0, seed: int = 0, n_targets: int = 1, balance_world: int = 0):
        self.rows, self.batch = rows, batch
        self.balance_world = int(balance_world)
        self.median, self.lmin, self.lmax = length_median, length_min, length_max
        self.alpha, self.sigma, self.seed, self.n_targets = zipf_alpha, sigma, seed, n_targets

    def _zipf(self, rng: np.random.Generator, n: int) -> np.ndarray:
        # inverse-CDF sample of a bounded Zipf: P(k) ~ k^-a on [1, rows]
        a = self.alpha
        u = rng.random(n)
        if abs(a - 1.0) < 1e-9:
            k = np.exp(u * np.log(self.rows))
        else:
            hi = self.rows ** (1.0 - a)
            k = (1.0 + u * (hi - 1.0)) ** (1.0 / (1.0 - a))
        return np.clip(k.astype(np.int64) - 1, 0, self.rows - 1)

    def batch_at(self, step: int, rank: int = 0, pin: bool = False) -> dict:
        rng = np.random.default_rng((self.seed * 1000003 + step) * 4099 + rank)
        if self.balance_world > 1:
            W = self.balance_world
            grng = np.random.default_rng((self.seed * 1000003 + step) * 4099 + 4098)      # the same draw on every rank
            allh = np.clip(np.exp(grng.normal(np.log(self.median), self.sigma, self.batch * W)), self.lmin,
                           self.lmax - self.n_targets).astype(np.int64)
            # longest first, each user to the least loaded rank that still has a free slot (cost = squared length)
            load = np.zeros(W)
            slots = np.full(W, self.batch)
            mine = []
            for h in allh[np.argsort(-allh, kind="stable")]:
                r = int(np.argmin(np.where(slots > 0, load, np.inf)))
                load[r] += float(h + self.n_targets) ** 2
                slots[r] -= 1
                if r == rank % W:
                    mine.append(h)
            hist = np.asarray(mine, dtype=np.int64)[rng.permutation(self.batch)]   # no length trend inside the rank's batch
        else:
            hist = np.clip(np.exp(rng.normal(np.log(self.median), self.sigma, self.batch)), self.lmin,
                           self.lmax - self.n_targets).astype(np.int64)
        lens = hist + self.n_targets
        offsets = np.zeros(self.batch + 1, dtype=np.int32)
        offsets[1:] = np.cumsum(lens)
        total = int(offsets[-1])
        ids = self._zipf(rng, total)
        ts = np.zeros(total, dtype=np.int64)
        actions = rng.integers(0, 8, total, dtype=np.int64)
        for b in range(self.batch):
            lo, hi = offsets[b], offsets[b + 1]
            gaps = rng.integers(1, 3600, hi - lo)
            ts[lo:hi] = 1_600_000_000 + np.cumsum(gaps)
        tgt = np.concatenate([np.arange(offsets[b + 1] - self.n_targets, offsets[b + 1]) for b in range(self.batch)])
        # learnable label: "listen-plus" (bit 1) on targets is a noisy function of the item id
        pos = ((ids[tgt] * 2654435761) >> 7) % 4 < 2
        flip = rng.random(len(tgt)) < 0.1
        actions[tgt] = (actions[tgt] & ~1) | (pos ^ flip).astype(np.int64)
        rows_pad = (total + 127) // 128 * 128
        out = {"offsets": torch.from_numpy(offsets), "num_targets": torch.full((self.batch,), self.n_targets, dtype=torch.int32),
               "timestamps": torch.from_numpy(ts), "actions": torch.from_numpy(actions), "item_ids": torch.from_numpy(ids),
               "total": total, "rows": rows_pad, "lengths": torch.from_numpy(lens), "max_targets": int(self.n_targets)}
        if pin and torch.cuda.is_available():
            out = {k: (v.pin_memory() if torch.is_tensor(v) else v) for k, v in out.items()}
        return out

    @staticmethod
    def to_device(batch: dict, device) -> dict:
        return {k: (v.to(device, non_blocking=True) if hasattr(v, "to") else v) for k, v in batch.items()}


def yambda_features(b: dict, tables: dict, uid: torch.Tensor, artist_of: torch.Tensor | None = None,
                    album_of: torch.Tensor | None = None) -> dict:
    """``b`` (item ids, offsets, targets of a batch) plus the keyed jagged features of the Yambda table set: per token the
    item, its artist and its album (``artist_of`` / ``album_of``: item -> id maps; without them an arithmetic map), per
    sample the user id and seven hashed crosses of the user with the item / artist / album it met last.  Adds
    ``samples`` (history features ``uih_*`` and candidate features) and ``token_row`` (row of every token inside the
    [history rows | candidate rows] concatenation the lookups return).  ``tables``: ``{name: TableConfig}`` - the row
    counts bound the ids."""
    from .samples import KeyedJagged, Samples, hashed_cross
    rows = {n: t.rows for n, t in tables.items()}
    item = b["item_ids"] % rows["item_id"]
    artist = (artist_of[b["item_ids"]] % rows["artist_id"] if artist_of is not None else item * 2654435761 % rows["artist_id"]).long()
    album = (album_of[b["item_ids"]] % rows["album_id"] if album_of is not None else item * 40503 % rows["album_id"]).long()
    offsets, nt = b["offsets"].long(), b["num_targets"].long()
    B = nt.numel()
    lens = offsets[1:] - offsets[:-1]
    pos = torch.arange(int(b["total"]))
    seq = torch.repeat_interleave(torch.arange(B), lens)
    is_cand = (pos - offsets[:-1][seq]) >= (lens - nt)[seq]
    hist_idx, cand_idx = torch.nonzero(~is_cand)[:, 0], torch.nonzero(is_cand)[:, 0]
    uid = uid.long() % rows["uid"]
    last_hist = (offsets[1:] - nt - 1).clamp(min=0)
    crosses = {}
    for k, other in enumerate((item, artist, album, item, artist, album, item)):
        name = f"cross_{k}"
        if name in rows:
            crosses[name] = hashed_cross(uid, other[last_hist] + k, rows[name], salt=k)
    one = torch.ones(B, dtype=torch.int64)
    uih = KeyedJagged.from_dict({"uih_item_id": (item[hist_idx], lens - nt), "uih_artist_id": (artist[hist_idx], lens - nt),
                                 "uih_album_id": (album[hist_idx], lens - nt), "uid": (uid, one),
                                 **{n: (v, one) for n, v in crosses.items()}})
    cand = KeyedJagged.from_dict({"item_id": (item[cand_idx], nt), "artist_id": (artist[cand_idx], nt),
                                  "album_id": (album[cand_idx], nt)})
    tok_row = torch.empty(int(b["total"]), dtype=torch.int64)
    tok_row[hist_idx] = torch.arange(hist_idx.numel())
    tok_row[cand_idx] = hist_idx.numel() + torch.arange(cand_idx.numel())
    return dict(b, samples=Samples(uih, cand, {}), token_row=tok_row)


class YambdaSyntheticSamples(HSTUSyntheticData):
    """Synthetic batches with the feature set of the Yambda benchmark tables: per token an item, its artist and its
    album; per sample a user id and hashed crosses of the user with what it listened to last - as a ``Samples`` of two
    keyed jagged tensors (history features ``uih_*``, candidate features) beside the dense payload, the structure the
    reference's loaders hand to the model (generative_recommenders/dlrm_v4/datasets/dataset.py ``Samples``;
    tables at generative_recommenders/dlrm_v4/configs.py:761-803).  ``tables``: ``TableConfig``s (row counts bound the ids)."""

    def __init__(self, tables, batch: int, **kw):
        self.tables = {t.name: t for t in tables}
        super().__init__(self.tables["item_id"].rows, batch, **kw)

    def batch_at(self, step: int, rank: int = 0, pin: bool = False) -> dict:
        b = super().batch_at(step, rank, pin=False)
        g = torch.Generator().manual_seed((self.seed * 1000003 + step) * 4099 + rank + 17)
        uid = torch.randint(0, self.tables["uid"].rows, (b["num_targets"].numel(),), generator=g)
        out = yambda_features(b, self.tables, uid)
        if pin and torch.cuda.is_available():
            out = {k: (v.pin_memory() if hasattr(v, "pin_memory") else v) for k, v in out.items()}
        return out

    @staticmethod
    def to_device(batch: dict, device) -> dict:
        return {k: (v.to(device, non_blocking=True) if hasattr(v, "to") else v) for k, v in batch.items()}
