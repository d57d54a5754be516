"""Token datasets for the LLM workloads.

* ``MMapIndexedDataset`` / ``write_indexed_dataset``: the Megatron ``.bin`` + ``.idx`` pair (index
  header ``MMIDIDX\\0\\0``, version 1, dtype code, sequence sizes, byte pointers, document index),
  memory-mapped, which is what the reference trains from
  (small_llm_pretraining/primus/conf/llama3.1_8B-pretrain-fp4.yaml:65-73 ``mmap`` bins of C4).
* ``GPTSampleDataset``: fixed-length ``seq_len + 1`` samples cut from the concatenated token stream
  of one or several weighted prefixes, with a seeded shuffle and deterministic rank/step slicing so
  a resumed run reads exactly the samples it would have read.
* ``PackedSFTDataset``: packed-sequence ``.npy`` files with a loss mask (the GovReport layout of
  llama2_sft/primus/scripts/convert_dataset.py: ``input_ids``, ``loss_mask``, ``seq_start_id``).
* ``SyntheticTokens``: uniform ids, the benchmark's stand-in stream.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np
import torch

_MAGIC = b"MMIDIDX\x00\x00"
_DTYPES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float32, 7: np.float64, 8: np.uint16}
_CODES = {np.dtype(v): k for k, v in _DTYPES.items()}


def write_indexed_dataset(prefix: str, documents: list[np.ndarray], dtype=np.int32) -> None:
    """Write ``prefix.bin`` / ``prefix.idx`` from a list of 1-D token arrays (one per document)."""
    dtype = np.dtype(dtype)
    sizes = np.array([len(d) for d in documents], dtype=np.int32)
    pointers = np.zeros(len(documents), dtype=np.int64)
    if len(documents) > 1:
        pointers[1:] = np.cumsum(sizes[:-1].astype(np.int64) * dtype.itemsize)
    with open(prefix + ".bin", "wb") as f:
        for d in documents:
            f.write(np.asarray(d, dtype=dtype).tobytes(order="C"))
    with open(prefix + ".idx", "wb") as f:
        f.write(_MAGIC)
        f.write(struct.pack("<Q", 1))
        f.write(struct.pack("<B", _CODES[dtype]))
        f.write(struct.pack("<Q", len(sizes)))
        f.write(struct.pack("<Q", len(sizes) + 1))
        f.write(sizes.tobytes(order="C"))
        f.write(pointers.tobytes(order="C"))
        f.write(np.arange(len(sizes) + 1, dtype=np.int64).tobytes(order="C"))


class MMapIndexedDataset:
    def __init__(self, prefix: str):
        with open(prefix + ".idx", "rb") as f:
            if f.read(9) != _MAGIC:
                raise ValueError(f"{prefix}.idx: not a Megatron index file")
            (version,) = struct.unpack("<Q", f.read(8))
            if version != 1:
                raise ValueError(f"{prefix}.idx: unsupported index version {version}")
            (code,) = struct.unpack("<B", f.read(1))
            (n,) = struct.unpack("<Q", f.read(8))
            (ndoc,) = struct.unpack("<Q", f.read(8))
            offset = f.tell()
        self.dtype = np.dtype(_DTYPES[code])
        idx = np.memmap(prefix + ".idx", mode="r", order="C")
        self.sizes = np.frombuffer(idx, dtype=np.int32, count=n, offset=offset)
        self.pointers = np.frombuffer(idx, dtype=np.int64, count=n, offset=offset + self.sizes.nbytes)
        self.doc_idx = np.frombuffer(idx, dtype=np.int64, count=ndoc, offset=offset + self.sizes.nbytes + self.pointers.nbytes)
        self.data = np.memmap(prefix + ".bin", mode="r", order="C")

    def __len__(self) -> int:
        return len(self.sizes)

    def __getitem__(self, i: int) -> np.ndarray:
        return np.frombuffer(self.data, dtype=self.dtype, count=int(self.sizes[i]), offset=int(self.pointers[i]))

    @property
    def num_tokens(self) -> int:
        return int(self.sizes.astype(np.int64).sum())

    def tokens(self, start: int, count: int) -> np.ndarray:
        """``count`` tokens of the concatenated stream starting at token ``start`` (documents are
        stored back to back in the .bin file, so this is one contiguous read)."""
        return np.frombuffer(self.data, dtype=self.dtype, count=count, offset=start * self.dtype.itemsize)


class GPTSampleDataset:
    """``seq_len + 1`` token windows over the concatenated streams of weighted prefixes.

    Sample ``i`` of the (seeded, shuffled) epoch order is a pure function of ``(seed, i)``: that is
    what makes mid-run resume exact.  ``batch(step, rank, world, local_batch)`` returns this rank's
    slice of global step ``step``."""

    def __init__(self, prefixes: list[str], weights: list[float] | None, seq_len: int, seed: int = 0):
        self.sets = [MMapIndexedDataset(p) for p in prefixes]
        w = np.array(weights if weights else [1.0] * len(self.sets), dtype=np.float64)
        self.weights = w / w.sum()
        self.seq_len = seq_len
        self.per_set = [max((s.num_tokens - 1) // seq_len, 0) for s in self.sets]
        self.total = int(sum(self.per_set))
        if self.total == 0:
            raise ValueError("dataset shorter than one sample")
        # a prefix shorter than one sample contributes nothing, whatever its weight
        self.weights = np.where(np.array(self.per_set) > 0, self.weights, 0.0)
        self.weights = self.weights / self.weights.sum()
        self.seed = seed
        # blended order: set index per sample drawn by weight, then a running cursor per set
        rng = np.random.default_rng(seed)
        choice = rng.choice(len(self.sets), size=self.total, p=self.weights)
        self.order_set = choice.astype(np.int32)
        self.order_idx = np.zeros(self.total, dtype=np.int64)
        for s in range(len(self.sets)):
            pos = np.nonzero(choice == s)[0]
            perm = rng.permutation(self.per_set[s]) if self.per_set[s] else np.zeros(0, dtype=np.int64)
            self.order_idx[pos] = perm[np.arange(len(pos)) % max(self.per_set[s], 1)] if self.per_set[s] else 0

    def __len__(self) -> int:
        return self.total

    def sample(self, i: int) -> np.ndarray:
        i %= self.total
        s, j = int(self.order_set[i]), int(self.order_idx[i])
        return self.sets[s].tokens(j * self.seq_len, self.seq_len + 1).astype(np.int64)

    def batch(self, step: int, rank: int, world: int, local_batch: int) -> torch.Tensor:
        base = (step * world + rank) * local_batch
        arr = np.stack([self.sample(base + k) for k in range(local_batch)])
        return torch.from_numpy(arr)


class PackedSFTDataset:
    """Packed fine-tuning samples: ``.npy`` object array of dicts with ``input_ids``, ``loss_mask``
    (1 where the token contributes to the loss) and ``seq_start_id`` (boundaries of the packed
    documents), plus an optional ``packed_metadata.jsonl``."""

    def __init__(self, npy_path: str, seq_len: int, metadata_path: str | None = None, pad_id: int = 0):
        self.rows = np.load(npy_path, allow_pickle=True)
        self.seq_len = seq_len
        self.pad_id = pad_id
        self.metadata = []
        if metadata_path and Path(metadata_path).exists():
            self.metadata = [json.loads(l) for l in Path(metadata_path).read_text().splitlines() if l.strip()]

    def __len__(self) -> int:
        return len(self.rows)

    def __getitem__(self, i: int):
        row = self.rows[i % len(self.rows)]
        ids = np.asarray(row["input_ids"], dtype=np.int64)[: self.seq_len + 1]
        mask = np.asarray(row.get("loss_mask", np.ones_like(ids)), dtype=np.int64)[: self.seq_len + 1]
        if len(ids) < self.seq_len + 1:
            pad = self.seq_len + 1 - len(ids)
            ids = np.concatenate([ids, np.full(pad, self.pad_id, dtype=np.int64)])
            mask = np.concatenate([mask, np.zeros(pad, dtype=np.int64)])
        tokens, labels = ids[:-1], ids[1:].copy()
        labels[mask[1:] == 0] = -100
        starts = np.asarray(row.get("seq_start_id", [0]), dtype=np.int64)
        return torch.from_numpy(tokens.copy()), torch.from_numpy(labels), torch.from_numpy(starts)

    def batch(self, step: int, rank: int, world: int, local_batch: int):
        base = (step * world + rank) * local_batch
        items = [self[base + k] for k in range(local_batch)]
        return torch.stack([t for t, _, _ in items]), torch.stack([l for _, l, _ in items])


def write_packed_sft(npy_path: str, samples: list[dict], metadata_path: str | None = None) -> None:
    arr = np.empty(len(samples), dtype=object)
    for i, s in enumerate(samples):
        arr[i] = s
    np.save(npy_path, arr, allow_pickle=True)
    if metadata_path:
        with open(metadata_path, "w") as f:
            for s in samples:
                f.write(json.dumps({"num_tokens": int(len(s["input_ids"])),
                                    "num_sequences": int(len(s.get("seq_start_id", [0])))}) + "\n")


class SyntheticTokens:
    """Uniform token ids, a pure function of ``(seed, step, rank)``."""

    def __init__(self, vocab: int, seq_len: int, seed: int = 0, loss_last: int = 0):
        self.vocab, self.seq_len, self.seed, self.loss_last = vocab, seq_len, seed, loss_last

    def batch(self, step: int, rank: int, world: int, local_batch: int) -> torch.Tensor:
        g = torch.Generator().manual_seed((self.seed * 1000003 + step) * 4099 + rank)
        return torch.randint(0, self.vocab, (local_batch, self.seq_len + 1), generator=g, dtype=torch.int64)

    def labels(self, tokens: torch.Tensor) -> torch.Tensor:
        """Next-token labels; with ``loss_last`` only the last N positions carry loss (the SFT
        benchmark variant: loss on the last 1024 positions)."""
        labels = tokens[:, 1:].clone()
        if self.loss_last > 0:
            labels[:, : labels.shape[1] - self.loss_last] = -100
        return labels
