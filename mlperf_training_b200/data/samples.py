"""Keyed jagged batches: the container every sparse feature of a recommender batch travels in.

``KeyedJagged`` holds, for a fixed list of feature keys, one flat ``values`` tensor and the per-key,
per-sample ``lengths`` (key-major: all samples of key 0, then key 1, ...), like TorchRec's
``KeyedJaggedTensor`` that the reference builds per batch
(generative_recommenders/dlrm_v4/datasets/dataset.py ``Samples``; merged user-history + candidate
tensors at generative_recommenders/modules/dlrm_hstu.py:1011-1017).  ``Samples`` pairs the
user-interaction-history features with the candidate features and the dense payload (timestamps,
action weights, watch time) of one batch; ``merged()`` is the single KJT a lookup consumes.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


class KeyedJagged:
    def __init__(self, keys: list[str], values: torch.Tensor, lengths: torch.Tensor):
        """``lengths``: int ``[len(keys) * batch]``, key-major; ``values``: ``[sum(lengths)]``."""
        if lengths.numel() % max(len(keys), 1):
            raise ValueError("lengths must hold one entry per key and sample")
        self.keys, self.values, self.lengths = list(keys), values, lengths
        self._offsets = None

    # ---- construction
    @staticmethod
    def from_dict(feats: dict[str, tuple[torch.Tensor, torch.Tensor]]) -> "KeyedJagged":
        """``{key: (values, lengths [batch])}`` -> one KJT (keys in dict order)."""
        keys = list(feats)
        return KeyedJagged(keys, torch.cat([feats[k][0] for k in keys]), torch.cat([feats[k][1] for k in keys]))

    @staticmethod
    def concat(parts: list["KeyedJagged"]) -> "KeyedJagged":
        """Keys of every part one after the other (the merged history + candidate tensor)."""
        keys = [k for p in parts for k in p.keys]
        if len(set(keys)) != len(keys):
            raise ValueError("duplicate feature keys in the parts of a merged batch")
        return KeyedJagged(keys, torch.cat([p.values for p in parts]), torch.cat([p.lengths for p in parts]))

    # ---- views
    @property
    def batch(self) -> int:
        return self.lengths.numel() // max(len(self.keys), 1)

    def offsets(self) -> torch.Tensor:
        if self._offsets is None:
            z = torch.zeros(1, dtype=torch.int64, device=self.lengths.device)
            self._offsets = torch.cat([z, torch.cumsum(self.lengths.long(), 0)])
        return self._offsets

    def key_ranges(self) -> dict[str, tuple[int, int]]:
        """Value range of every key (host integers: one read of the offsets)."""
        b = self.batch
        off = self.offsets()[:: b].tolist() if b else [0]
        return {k: (off[i], off[i + 1]) for i, k in enumerate(self.keys)}

    def __getitem__(self, key: str) -> tuple[torch.Tensor, torch.Tensor]:
        i = self.keys.index(key)
        b = self.batch
        lo, hi = int(self.offsets()[i * b]), int(self.offsets()[(i + 1) * b])
        return self.values[lo:hi], self.lengths[i * b:(i + 1) * b]

    def to(self, device, non_blocking: bool = False) -> "KeyedJagged":
        return KeyedJagged(self.keys, self.values.to(device, non_blocking=non_blocking),
                           self.lengths.to(device, non_blocking=non_blocking))

    def pin_memory(self) -> "KeyedJagged":
        return KeyedJagged(self.keys, self.values.pin_memory(), self.lengths.pin_memory())

    def permute(self, keys: list[str]) -> "KeyedJagged":
        return KeyedJagged.from_dict({k: self[k] for k in keys})


@dataclass
class Samples:
    """One batch: history features, candidate features, dense payload ``{name: jagged values}``."""
    uih: KeyedJagged
    candidates: KeyedJagged
    payload: dict = field(default_factory=dict)

    def merged(self) -> KeyedJagged:
        return KeyedJagged.concat([self.uih, self.candidates])

    def to(self, device, non_blocking: bool = False) -> "Samples":
        return Samples(self.uih.to(device, non_blocking), self.candidates.to(device, non_blocking),
                       {k: (v.to(device, non_blocking=non_blocking) if torch.is_tensor(v) else v) for k, v in self.payload.items()})

    def pin_memory(self) -> "Samples":
        return Samples(self.uih.pin_memory(), self.candidates.pin_memory(),
                       {k: (v.pin_memory() if torch.is_tensor(v) else v) for k, v in self.payload.items()})


def hashed_cross(a: torch.Tensor, b: torch.Tensor, rows: int, salt: int = 0) -> torch.Tensor:
    """Id of the crossed feature ``(a, b)`` in a hashed table of ``rows`` rows: a 64-bit mix of the two ids
    reduced modulo the table size (the hashed user x item / artist / album crosses of the Yambda feature
    set, generative_recommenders/dlrm_v4/configs.py:761-803)."""
    m = (1 << 63) - 1
    x = (a.long() * 0x9E3779B97F4A7C15 + salt) & m
    x = (x ^ (x >> 31)) * 0x7FB5D329728EA185 & m
    x = (x ^ (b.long() * 0x94D049BB133111EB & m)) & m
    x = (x ^ (x >> 29)) & m
    return x % rows
