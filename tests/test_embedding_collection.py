"""Keyed jagged batches, hashed crosses, the table planner and the multi-table lookup (CPU; a gloo
world of 2 checks table-wise and row-wise placement against an unsharded copy)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mlperf_training_b200.data.samples import KeyedJagged, Samples, hashed_cross
from mlperf_training_b200.parallel.embedding_collection import (YAMBDA_TABLES, EmbeddingCollection, TableConfig, plan_tables)


def test_keyed_jagged_round_trip():
    a = (torch.tensor([3, 4, 5]), torch.tensor([2, 1]))
    b = (torch.tensor([7]), torch.tensor([0, 1]))
    k = KeyedJagged.from_dict({"a": a, "b": b})
    assert k.batch == 2 and k.key_ranges() == {"a": (0, 3), "b": (3, 4)}
    assert torch.equal(k["b"][0], torch.tensor([7])) and torch.equal(k["a"][1], torch.tensor([2, 1]))
    s = Samples(k, KeyedJagged.from_dict({"c": (torch.tensor([9, 9]), torch.tensor([1, 1]))}), {"ts": torch.arange(4)})
    m = s.merged()
    assert m.keys == ["a", "b", "c"] and m.values.tolist() == [3, 4, 5, 7, 9, 9]
    assert m.permute(["c", "a"]).values.tolist() == [9, 9, 3, 4, 5]
    with pytest.raises(ValueError):
        KeyedJagged.concat([k, k])


def test_hashed_cross_is_deterministic_and_spread():
    u = torch.arange(1000).repeat_interleave(10)
    i = torch.arange(10).repeat(1000)
    h = hashed_cross(u, i, 4096, salt=3)
    assert torch.equal(h, hashed_cross(u, i, 4096, salt=3)) and int(h.min()) >= 0 and int(h.max()) < 4096
    assert not torch.equal(h, hashed_cross(u, i, 4096, salt=4))
    counts = torch.bincount(h, minlength=4096).float()
    assert counts.max() < 6 * counts.mean()


def test_planner_places_big_tables_row_wise_and_balances_the_rest():
    plan = plan_tables(YAMBDA_TABLES, 8, row_wise_min_bytes=4 << 30)
    assert plan["cross_0"] == ("row_wise", None) and plan["item_id"] == ("row_wise", None)       # 100 M x 512 bf16, 9.4 M x 512
    assert plan["uid"][0] == "table_wise" and plan["artist_id"][0] == "table_wise" and plan["cross_5"][0] == "table_wise"
    owners = [v[1] for v in plan.values() if v[0] == "table_wise"]
    assert len(set(owners)) == len(owners)                                                      # small tables on different ranks
    with pytest.raises(MemoryError):
        plan_tables(YAMBDA_TABLES, 8, budget_bytes=1 << 30)
    assert all(v == ("row_wise", None) for v in plan_tables(YAMBDA_TABLES, 1).values())


def _tables():
    return [TableConfig("item", 64, 8, ("uih_item", "item"), "fp32"), TableConfig("uid", 16, 8, ("uid",), "fp32"),
            TableConfig("cross", 40, 8, ("cross",), "fp32")]


def _kjt(seed):
    g = torch.Generator().manual_seed(seed)
    return KeyedJagged.from_dict({"uih_item": (torch.randint(0, 64, (9,), generator=g), torch.tensor([4, 5])),
                                  "item": (torch.randint(0, 64, (2,), generator=g), torch.tensor([1, 1])),
                                  "uid": (torch.randint(0, 16, (2,), generator=g), torch.tensor([1, 1])),
                                  "cross": (torch.randint(0, 40, (2,), generator=g), torch.tensor([1, 1]))})


def test_collection_lookup_and_update_single_rank():
    ec = EmbeddingCollection(_tables(), lr=0.5, seed=1)
    k = _kjt(0)
    out = ec.lookup(k)
    assert set(out) == {"uih_item", "item", "uid", "cross"} and out["uih_item"].shape == (9, 8)
    w0 = ec.tables["item"].weight.clone()
    assert torch.equal(out["item"], w0[k["item"][0]])
    sum(v.sum() for v in out.values()).backward()
    assert not torch.equal(ec.tables["item"].weight, w0)
    sd = ec.state_dict()
    assert "embeddings.uid.weight" in sd and sd["embeddings.cross.weight.global_rows"] == 40
    ec2 = EmbeddingCollection(_tables(), seed=9)
    ec2.load_state_dict(sd)
    assert torch.equal(ec2.tables["uid"].weight, ec.tables["uid"].weight)


def _worker(rank, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=2)
    try:
        plan = {"item": ("row_wise", None), "uid": ("table_wise", 1), "cross": ("table_wise", 0)}
        ec = EmbeddingCollection(_tables(), lr=0.5, seed=1, plan=plan)
        # the unsharded truth: gather every table
        full = {}
        for name, t in ec.tables.items():
            parts = [torch.zeros(t.rows, t.dim) for _ in range(2)]
            mine = torch.zeros(t.rows, t.dim)
            mine[t.row_lo:t.row_lo + t.local_rows] = t.weight
            dist.all_gather(parts, mine)
            full[name] = parts[0] + parts[1]
        k = _kjt(rank)
        out = ec.lookup(k)
        ok = all(torch.equal(out[f], full[ec.feature_table[f]][k[f][0]]) for f in out)
        ok &= ec.tables["uid"].local_rows == (16 if rank == 1 else 0) and ec.tables["cross"].local_rows == (40 if rank == 0 else 0)
        sum(v.sum() for v in out.values()).backward()                     # sparse updates reach the owners
        moved = torch.tensor([float((ec.tables["uid"].weight != full["uid"][ec.tables["uid"].row_lo:ec.tables["uid"].row_lo + ec.tables["uid"].local_rows]).any())
                              if rank == 1 else 1.0])
        dist.all_reduce(moved, op=dist.ReduceOp.MIN)
        q.put((rank, bool(ok) and bool(moved.item() > 0)))
    finally:
        dist.destroy_process_group()


def test_collection_table_wise_and_row_wise_gloo():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res == {0: True, 1: True}


def test_sharded_state_round_trips_across_placement_plans_gloo(tmp_path):
    """TorchRec-layout sharded state: written row-wise / table-wise by 2 ranks, read back under the same and under the
    swapped placement plan."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=root)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29655",
                        os.path.join(root, "tests", "multi", "emb_ckpt_worker.py"), str(tmp_path)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("ok=True") == 2


def _cw_worker(rank, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=2)
    try:
        tabs = [TableConfig("wide", 40, 8, ("wide",), "fp32")]
        ec = EmbeddingCollection(tabs, lr=0.5, seed=3, plan=plan_tables(tabs, 2, column_wise=("wide",)))
        t = ec.tables["wide"]
        ok = t.weight.shape == (40, 4) and t.col_lo == 4 * rank
        parts = [torch.zeros(40, 4) for _ in range(2)]
        dist.all_gather(parts, t.weight.clone())
        full = torch.cat(parts, 1)
        g = torch.Generator().manual_seed(10 + rank)
        ids = torch.randint(0, 40, (11,), generator=g)
        ids[3] = ids[0]                                                     # a duplicate on this rank
        out = ec.lookup(KeyedJagged.from_dict({"wide": (ids, torch.tensor([5, 6]))}))["wide"]
        ok &= torch.equal(out, full[ids])
        coef = torch.randn(11, 8, generator=g)
        (out * coef).sum().backward()
        # the unsharded truth: both ranks' gradient rows summed per id; Adagrad sum per column shard
        both_ids, both_g = [torch.zeros(11, dtype=torch.int64) for _ in range(2)], [torch.zeros(11, 8) for _ in range(2)]
        dist.all_gather(both_ids, ids)
        dist.all_gather(both_g, coef)
        dense = torch.zeros(40, 8).index_add_(0, torch.cat(both_ids), torch.cat(both_g))
        hit = torch.zeros(40, dtype=torch.bool)
        hit[torch.cat(both_ids)] = True
        mine = dense[:, 4 * rank:4 * rank + 4]
        st = (mine * mine).mean(-1)
        want = full[:, 4 * rank:4 * rank + 4] - 0.5 * mine / (st.sqrt()[:, None] + 1e-8)
        want = torch.where(hit[:, None], want, full[:, 4 * rank:4 * rank + 4])
        ok &= torch.allclose(t.weight, want, atol=1e-6) and torch.allclose(t.state, torch.where(hit, st, torch.zeros(())), atol=1e-6)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_column_wise_table_lookup_and_update_gloo():
    """COLUMN_WISE: every rank holds half the width of every row; rows come back whole, the sparse update
    reaches both column shards with the gradient rows of both ranks."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_cw_worker, args=(r, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res == {0: True, 1: True}


def test_column_wise_single_rank_is_a_plain_table():
    from mlperf_training_b200.parallel.embedding import ColumnShardedEmbedding
    t = ColumnShardedEmbedding(20, 6, dtype=torch.float32, lr=0.1, seed=2)
    ids = torch.tensor([3, 3, 7])
    w0 = t.weight.clone()
    rows = t.lookup(ids)
    assert torch.equal(rows, w0[ids])
    rows.sum().backward()
    assert not torch.equal(t.weight[3], w0[3]) and torch.equal(t.weight[4], w0[4])
    with pytest.raises(ValueError):
        plan_tables([TableConfig("odd", 10, 7, ("odd",))], 2, column_wise=("odd",))
