"""Embedding collection: many named tables, each sharded by a planner, looked up from one keyed jagged batch.

``plan_tables`` decides per table between ROW_WISE (rows cut evenly over the ranks: the big tables),
TABLE_WISE (the whole table on one rank, ranks filled greedily by bytes: the small ones) and, for the
tables a caller names, COLUMN_WISE (every rank holds a slice of the width of every row) under a
per-rank memory budget - the decision TorchRec's planner makes for the reference
(generative_recommenders/dlrm_v4/train/utils.py:1311-1545; tables at
generative_recommenders/dlrm_v4/configs.py:761-803).  ``EmbeddingCollection.lookup`` takes a
``KeyedJagged`` batch, issues ONE lookup per table over the concatenated ids of all features that
read the table, and returns ``{feature: rows}``; backward applies each table's row-wise Adagrad.
The state dict exposes every shard under ``embeddings.<table>.weight`` with its row offset.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..data.samples import KeyedJagged
from .embedding import ColumnShardedEmbedding, ShardedEmbedding


@dataclass
class TableConfig:
    name: str
    rows: int
    dim: int
    features: tuple          # feature keys that read this table
    dtype: str = "bf16"

    def bytes(self) -> int:
        return self.rows * self.dim * (2 if self.dtype == "bf16" else 4)


# the Yambda-5b feature set of the DLRMv4 benchmark: ids, user id and seven hashed crosses, width 512
YAMBDA_TABLES = (
    TableConfig("item_id", 9_390_624, 512, ("uih_item_id", "item_id")),
    TableConfig("artist_id", 1_293_395, 512, ("uih_artist_id", "artist_id")),
    TableConfig("album_id", 3_367_692, 512, ("uih_album_id", "album_id")),
    TableConfig("uid", 1_000_001, 512, ("uid",)),
    TableConfig("cross_0", 100_000_000, 512, ("cross_0",)),
    TableConfig("cross_1", 40_000_000, 512, ("cross_1",)),
    TableConfig("cross_2", 24_000_000, 512, ("cross_2",)),
    TableConfig("cross_3", 40_000_000, 512, ("cross_3",)),
    TableConfig("cross_4", 32_000_000, 512, ("cross_4",)),
    TableConfig("cross_5", 2_000_000, 512, ("cross_5",)),
    TableConfig("cross_6", 40_000_000, 512, ("cross_6",)),
)


def plan_tables(tables, world: int, row_wise_min_bytes: int = 1 << 30, budget_bytes: int | None = None,
                column_wise: tuple = ()) -> dict:
    """``{table: ("row_wise", None) | ("table_wise", owner) | ("column_wise", None)}``.  Tables named in
    ``column_wise`` (their width must divide by the ranks) are cut along columns; tables of at least
    ``row_wise_min_bytes`` are cut over all ranks by rows; the others go whole to the rank that holds the
    fewest bytes so far (largest first).  With ``budget_bytes`` the plan is checked against a per-rank limit."""
    out, load = {}, [0] * max(world, 1)
    small = []
    for t in tables:
        if world > 1 and t.name in column_wise:
            if t.dim % world:
                raise ValueError(f"table {t.name}: width {t.dim} does not divide by {world} ranks")
            out[t.name] = ("column_wise", None)
            for r in range(world):
                load[r] += t.bytes() // world
        elif world > 1 and t.bytes() >= row_wise_min_bytes:
            out[t.name] = ("row_wise", None)
            for r in range(world):
                load[r] += t.bytes() // world
        else:
            small.append(t)
    for t in sorted(small, key=lambda t: -t.bytes()):
        r = min(range(len(load)), key=lambda i: load[i])
        out[t.name] = ("table_wise", r) if world > 1 else ("row_wise", None)
        load[r] += t.bytes()
    if budget_bytes is not None and max(load) > budget_bytes:
        raise MemoryError(f"embedding plan needs {max(load) / 2**30:.1f} GiB on a rank, budget {budget_bytes / 2**30:.1f} GiB")
    return out


class EmbeddingCollection:
    def __init__(self, tables, *, group=None, device="cpu", lr: float = 1e-2, eps: float = 1e-8, seed: int = 0,
                 comm: str = "nccl", plan: dict | None = None, row_wise_min_bytes: int = 1 << 30, scale_rows: int = 1):
        """``scale_rows`` divides every table's row count (smoke runs of the full feature set)."""
        self.configs = [TableConfig(t.name, max(t.rows // scale_rows, 2), t.dim, tuple(t.features), t.dtype) for t in tables]
        world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.plan = plan or plan_tables(self.configs, world, row_wise_min_bytes)
        self.tables: dict[str, ShardedEmbedding] = {}
        self.feature_table: dict[str, str] = {}
        for i, t in enumerate(self.configs):
            kind, owner = self.plan[t.name]
            dt = torch.bfloat16 if t.dtype == "bf16" else torch.float32
            cls = ColumnShardedEmbedding if kind == "column_wise" else ShardedEmbedding
            self.tables[t.name] = cls(t.rows, t.dim, group=group, device=device, dtype=dt, lr=lr, eps=eps,
                                      seed=seed + 101 * i, comm=comm if kind == "row_wise" else "nccl", name=t.name,
                                      owner=owner if kind == "table_wise" else None)
            for f in t.features:
                self.feature_table[f] = t.name

    def set_lr(self, lr: float) -> None:
        for t in self.tables.values():
            t.lr = lr

    @property
    def lr(self) -> float:
        return next(iter(self.tables.values())).lr

    @lr.setter
    def lr(self, value: float) -> None:
        self.set_lr(value)

    def snapshot(self):
        return {n: t.snapshot() for n, t in self.tables.items()}

    def restore(self, snap) -> None:
        for n, t in self.tables.items():
            t.restore(snap[n])

    def lookup(self, kjt: KeyedJagged) -> dict[str, torch.Tensor]:
        """``{feature: rows [n_values(feature), dim]}`` for every key of ``kjt`` that maps to a table."""
        ranges = kjt.key_ranges()
        by_table: dict[str, list[str]] = {}
        for k in kjt.keys:
            if k in self.feature_table:
                by_table.setdefault(self.feature_table[k], []).append(k)
        out = {}
        for name, keys in by_table.items():
            ids = torch.cat([kjt.values[ranges[k][0]:ranges[k][1]] for k in keys])
            rows = self.tables[name].lookup(ids)
            pos = 0
            for k in keys:
                n = ranges[k][1] - ranges[k][0]
                out[k] = rows[pos:pos + n]
                pos += n
        return out

    def state_dict(self) -> dict:
        sd = {}
        for t in self.tables.values():
            sd.update(t.state_dict())
        return sd

    def load_state_dict(self, sd: dict) -> None:
        for t in self.tables.values():
            t.load_state_dict(sd)

    def sharded_state_dict(self, prefix: str = "") -> dict:
        """Every table as ``ShardedTensor``s under TorchRec's key names (see ``ShardedEmbedding.sharded_state_dict``)."""
        sd = {}
        for t in self.tables.values():
            sd.update(t.sharded_state_dict(prefix))
        return sd

    def save_sharded(self, path: str, prefix: str = "") -> None:
        import torch.distributed.checkpoint as dcp
        dcp.save(self.sharded_state_dict(prefix), checkpoint_id=str(path))

    def load_sharded(self, path: str, prefix: str = "") -> None:
        """Load a sharded checkpoint written under any number of ranks and any placement plan."""
        from .embedding import load_matching
        load_matching(self.sharded_state_dict(prefix), path)

    def local_bytes(self) -> int:
        return sum(t.weight.numel() * t.weight.element_size() for t in self.tables.values())
