"""HSTU workload on CPU: metrics, sharded embedding (single rank + gloo world 2), trainer run with
MLLOG compliance and a fault-injected resume."""
import io
import os
import subprocess
import sys

import pytest
import torch

from mlperf_training_b200.mllog import check_compliance
from mlperf_training_b200.parallel.embedding import ShardedEmbedding
from mlperf_training_b200.utils.metrics import BinnedCumulativeAUC, exact_auc, normalized_entropy

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _exp(**kw):
    e = dict(batch_per_gpu=8, train_steps=12, dense_lr=3e-3, sparse_lr=0.1, eval_interval_steps=6, num_eval_batches=2,
             model=dict(layers=2, dim=32, heads=2, d_qk=16, d_v=16, max_seq_len=48, dtype="fp32", mlp_hidden=16,
                        num_positions=64, num_time_buckets=32),
             embedding=dict(rows=200, dim=16), data=dict(length_median=12, length_min=4, length_max=40))
    e.update(kw)
    return e


def test_auc_matches_pair_counting():
    g = torch.Generator().manual_seed(0)
    s = torch.rand(200, generator=g).round(decimals=2)          # ties on purpose
    y = (torch.rand(200, generator=g) < 0.3).float()
    pos, neg = s[y == 1], s[y == 0]
    brute = ((pos[:, None] > neg[None]).double() + 0.5 * (pos[:, None] == neg[None]).double()).mean().item()
    assert abs(exact_auc(s, y) - brute) < 1e-12
    b = BinnedCumulativeAUC(bins=100)
    b.update(s[:100], y[:100])
    b.update(s[100:], y[100:])
    assert abs(b.compute() - brute) < 2e-2
    b2 = BinnedCumulativeAUC(bins=100)
    b2.load_state_dict(b.state_dict())
    assert b2.compute() == b.compute()
    assert exact_auc(s, torch.ones_like(y)) == 0.5
    assert normalized_entropy(torch.full((100,), float(y.mean())), y[:100]) > 0.9


def test_sharded_embedding_single_rank_adagrad():
    t = ShardedEmbedding(50, 8, dtype=torch.float32, lr=0.5, seed=1)
    w0 = t.weight.clone()
    ids = torch.tensor([3, 7, 3, 9])
    out = t.lookup(ids)
    assert torch.equal(out, w0[ids])
    out.sum().backward()
    g = torch.zeros(50, 8)
    g[3], g[7], g[9] = 2.0, 1.0, 1.0
    st = (g * g).mean(-1)
    ref = w0 - 0.5 * g / (st.sqrt()[:, None] + t.eps)
    assert torch.allclose(t.weight, ref, atol=1e-6)
    sd = t.state_dict()
    assert sd["embeddings.item.weight.row_offset"] == 0
    t2 = ShardedEmbedding(50, 8, dtype=torch.float32, seed=2)
    t2.load_state_dict(sd)
    assert torch.equal(t2.weight, t.weight)


def test_sharded_embedding_gloo_world2():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29631",
                        os.path.join(ROOT, "tests", "multi", "embedding_worker.py"), "gloo"],
                       env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


def test_hstu_run_learns_and_logs():
    from mlperf_training_b200.trainer.hstu import run
    out = run(_exp(train_steps=40, eval_interval_steps=20), device="cpu", stream=io.StringIO())
    assert out["losses"][-1] < out["losses"][0]
    assert out["aucs"][-1] > 0.6
    assert check_compliance(out["records"]) == []


@pytest.mark.parametrize("sparse_format", ["per_rank", "sharded"])
def test_hstu_die_and_resume(tmp_path, sparse_format):
    from mlperf_training_b200.trainer.hstu import run
    ref = run(_exp(), device="cpu", stream=io.StringIO())
    e = _exp(checkpoint_dir=str(tmp_path / "ck"), die_at_step=6, mllog_file=str(tmp_path / "ml.log"),
             sparse_checkpoint=sparse_format)
    with pytest.raises(SystemExit) as ex:
        run(e, device="cpu", stream=io.StringIO())
    assert ex.value.code == 42
    e["die_at_step"] = 0
    out = run(e, device="cpu", stream=io.StringIO())
    assert abs(out["losses"][-1] - ref["losses"][-1]) < 1e-5
    lines = open(tmp_path / "ml.log").read().splitlines()
    assert sum("run_start" in l for l in lines) == 1 and sum("run_stop" in l for l in lines) == 1
    # a resume that changes what the split or the stream position depends on is refused ...
    changed = dict(e, batch_per_gpu=int(e.get("batch_per_gpu", 4)) * 2, train_steps=int(e.get("train_steps", 8)) + 2)
    with pytest.raises(RuntimeError, match="split contract"):
        run(changed, device="cpu", stream=io.StringIO())


def test_split_contract_override(monkeypatch):
    from mlperf_training_b200.checkpoint.manager import validate_split_contract
    saved, live = {"salt": 1, "holdout": 0.1, "world": 8}, {"salt": 2, "holdout": 0.1, "world": 8}
    with pytest.raises(RuntimeError):
        validate_split_contract(saved, live)
    validate_split_contract(saved, live, allow_mismatch=True)          # ALLOW_SPLIT_MISMATCH=1
    validate_split_contract(None, live)                                # a checkpoint from before contracts were recorded


def test_hstu_lr_warmup_ramps_dense_and_sparse_rates():
    from mlperf_training_b200.models.hstu import tiny_hstu
    from mlperf_training_b200.trainer.hstu import HSTUTrainer
    tr = HSTUTrainer(tiny_hstu(), 200, 2, "cpu", dense_lr=1e-3, sparse_lr=1e-2, data_kw=dict(length_median=12, length_min=4, length_max=24))
    assert tr.lrs_at(0) == (1e-3, 1e-2)                                    # no warm-up configured
    tr.lr_warmup_steps, tr.lr_warmup_start_lr = 10, 5e-3                   # a floor above the dense base: dense does not ramp
    d0, s0 = tr.lrs_at(0)
    assert d0 == 1e-3 and s0 == 5e-3
    d5, s5 = tr.lrs_at(5)
    assert d5 == 1e-3 and abs(s5 - 7.5e-3) < 1e-12
    assert tr.lrs_at(10) == (1e-3, 1e-2) and tr.lrs_at(50) == (1e-3, 1e-2)
    tr.lr_warmup_start_lr = 0.0
    w0 = [p.detach().clone() for p in tr.model.parameters()]
    t0 = tr.table.weight.detach().clone()
    tr.train_step(0)                                                       # step 0 of a ramp from zero changes nothing
    assert all(torch.equal(a, b) for a, b in zip(w0, tr.model.parameters())) and torch.equal(t0, tr.table.weight)
    tr.train_step(1)
    assert any(not torch.equal(a, b) for a, b in zip(w0, tr.model.parameters())) and not torch.equal(t0, tr.table.weight)


def test_hstu_unpipelined_loop_gives_the_same_losses():
    from mlperf_training_b200.models.hstu import tiny_hstu
    from mlperf_training_b200.trainer.hstu import HSTUTrainer
    out = []
    for pipelined in (True, False):
        tr = HSTUTrainer(tiny_hstu(input_dropout=0.0, linear_dropout=0.0), 200, 2, "cpu", seed=1,
                         data_kw=dict(length_median=12, length_min=4, length_max=24))
        tr.pipelined = pipelined
        out.append([float(tr.train_step(i)) for i in range(3)])
    assert out[0] == out[1]


def test_eval_cadence_from_data_fractions():
    from mlperf_training_b200.trainer.cadence import data_pct_to_global_steps, first_eval_steps, should_eval, skip_eval_until_step
    assert data_pct_to_global_steps(0.01, 1_000_000, 1024) == 10                 # ceil(10000 / 1024)
    assert data_pct_to_global_steps(0.0, 10, 2) == 0 and data_pct_to_global_steps(0.5, 0, 2) == 0
    assert skip_eval_until_step(0.25, 1000, 10) == 25 and skip_eval_until_step(0.0, 1000, 10) == 0
    # the MLPerf rule at GBS 8192 over 300 M samples: interval 37 steps of 8192, first evaluation at the
    # first multiple of it at or after floor((4480 * 8192 + 135331840) / 3) samples
    gbs, total = 8192, 300_000_000
    interval = -(-int(0.001 * total) // gbs) * gbs
    first = (4480 * gbs + 135331840) // 3
    want = -(-first // interval) * interval // gbs
    assert skip_eval_until_step(-1.0, total, gbs) == want and want * gbs >= first
    assert first_eval_steps(0, 10, 0) == 10 and first_eval_steps(10, 10, 0) == 10 and first_eval_steps(3, 10, 25) == 27
    assert first_eval_steps(5, 0, 0) == 0
    assert [g for g in range(1, 41) if should_eval(g, 10, 25)] == [30, 40]
    assert not should_eval(0, 10) and not should_eval(10, 0)


def test_hstu_run_skips_early_evaluations():
    import io
    from mlperf_training_b200.trainer.hstu import run
    exp = dict(batch_per_gpu=2, train_steps=8, eval_interval_steps=0, num_eval_batches=1, total_train_samples=16,
               eval_every_data_pct=0.25, skip_eval_epoch_pct=0.5,
               model=dict(layers=1, dim=32, heads=2, d_qk=16, d_v=16, max_seq_len=32, dtype="fp32", mlp_hidden=16,
                          num_positions=64, num_time_buckets=32),
               embedding=dict(rows=300, dim=16), data=dict(length_median=10, length_min=4, length_max=24))
    out = run(exp, device="cpu", stream=io.StringIO())
    # 25 % of 16 samples at global batch 2 = every 2 steps; nothing before 50 % = step 4: evaluations after steps 4, 6, 8
    assert len(out["aucs"]) == 3


def test_length_balanced_placement_keeps_the_global_batch():
    """Dealing a step's users to the ranks by length changes placement only: the union over ranks is one draw of
    W x batch lengths, every rank gets `batch` users, and the squared-length cost per rank is nearly equal."""
    import numpy as np
    from mlperf_training_b200.data.hstu_synth import HSTUSyntheticData
    W, B = 4, 64
    d = HSTUSyntheticData(10 ** 5, B, seed=3, balance_world=W, length_median=200, length_max=2048)
    per_rank = [d.batch_at(5, r)["lengths"].numpy() for r in range(W)]
    assert all(len(x) == B for x in per_rank)
    again = [d.batch_at(5, r)["lengths"].numpy() for r in range(W)]
    assert all((a == b).all() for a, b in zip(per_rank, again))                       # deterministic per (step, rank)
    grng = np.random.default_rng((3 * 1000003 + 5) * 4099 + 4098)
    want = np.clip(np.exp(grng.normal(np.log(200), 1.0, B * W)), 16, 2048 - 1).astype(np.int64) + 1
    assert sorted(np.concatenate(per_rank).tolist()) == sorted(want.tolist())          # the same multiset of users
    cost = np.array([(x.astype(np.float64) ** 2).sum() for x in per_rank])
    plain = HSTUSyntheticData(10 ** 5, B, seed=3, length_median=200, length_max=2048)
    cost0 = np.array([(plain.batch_at(5, r)["lengths"].numpy().astype(np.float64) ** 2).sum() for r in range(W)])
    assert cost.max() / cost.mean() < 1.05 <= cost0.max() / cost0.mean() + 0.05


def test_multi_table_run_learns_and_resumes(tmp_path):
    """The benchmark's eleven-table feature set (item / artist / album ids, user id, seven hashed crosses) through the
    run loop: keyed jagged batches, one lookup per table, additional-feature branch and contextual tokens in the
    model; the loss falls, and a run that dies and resumes ends where the uninterrupted one does."""
    from mlperf_training_b200.trainer.hstu import run
    base = dict(embedding=dict(rows=200, dim=16, tables="yambda", table_scale=20000), train_steps=10, eval_interval_steps=0,
                num_eval_batches=0)
    ref = run(_exp(**base), device="cpu", stream=io.StringIO())
    assert ref["losses"][-1] < ref["losses"][0]
    e = _exp(checkpoint_dir=str(tmp_path / "ck"), die_at_step=5, sparse_checkpoint="sharded", **base)
    with pytest.raises(SystemExit) as ex:
        run(e, device="cpu", stream=io.StringIO())
    assert ex.value.code == 42
    e["die_at_step"] = 0
    out = run(e, device="cpu", stream=io.StringIO())
    assert abs(out["losses"][-1] - ref["losses"][-1]) < 1e-5


def test_yambda_synthetic_samples_are_consistent():
    from mlperf_training_b200.data.hstu_synth import YambdaSyntheticSamples
    from mlperf_training_b200.parallel.embedding_collection import TableConfig, YAMBDA_TABLES
    tables = [TableConfig(t.name, max(t.rows // 10000, 2), 8, t.features, "fp32") for t in YAMBDA_TABLES]
    d = YambdaSyntheticSamples(tables, 6, seed=1, length_median=10, length_min=3, length_max=30)
    b = d.batch_at(2, 0)
    s = b["samples"]
    kjt = s.merged()
    ranges = kjt.key_ranges()
    n_hist = int((b["lengths"] - b["num_targets"]).sum())
    assert ranges["uih_item_id"][1] - ranges["uih_item_id"][0] == n_hist
    assert ranges["item_id"][1] - ranges["item_id"][0] == int(b["num_targets"].sum())
    assert ranges["uid"][1] - ranges["uid"][0] == 6 and all(f"cross_{k}" in ranges for k in range(7))
    # token order: the [history | candidates] concatenation re-ordered by token_row gives back the flat item ids
    cat = torch.cat([kjt.values[slice(*ranges["uih_item_id"])], kjt.values[slice(*ranges["item_id"])]])
    assert torch.equal(cat[b["token_row"]], b["item_ids"])
    for t in tables:
        for f in t.features:
            assert int(kjt.values[slice(*ranges[f])].max()) < t.rows


def test_hstu_trainer_steps_with_the_interleaved_preprocessor():
    from mlperf_training_b200.models.hstu import tiny_hstu
    from mlperf_training_b200.trainer.hstu import HSTUTrainer
    tr = HSTUTrainer(tiny_hstu(preprocessor="interleave", input_dropout=0.0, linear_dropout=0.0), 200, 3, "cpu", seed=2,
                     data_kw=dict(length_median=12, length_min=4, length_max=24))
    losses = [float(tr.train_step(i)) for i in range(4)]
    assert all(l == l and l < 10 for l in losses)


def test_hstu_loop_with_column_wise_tables_resumes_gloo(tmp_path):
    """Two ranks, the eleven-table set with two tables cut along their width: the loop trains, writes the sharded
    sparse checkpoint, exits, and the resumed run continues on the straight run's losses."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29678",
                        os.path.join(ROOT, "tests", "multi", "hstu_loop_worker.py"), str(tmp_path)],
                       env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("ok=True") == 2


def test_experiment_file_reaches_every_model_field():
    """Stochastic depth, recent-window layers, the postprocessor and the task list are set from the ``model`` section of
    an experiment; a key that means nothing is reported, not silently dropped."""
    import warnings
    from mlperf_training_b200.trainer.hstu import run
    e = _exp(train_steps=3, eval_interval_steps=0, num_eval_batches=0)
    e["model"] = dict(e["model"], layers=3, sd_ratio=0.5, recent_window=8, recent_window_layers=1, postprocessor="l2",
                      input_dropout=0.0, tasks=[["listen_plus", 1, "binary"], ["like", 2, "binary"]], bogus=1)
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        out = run(e, device="cpu", stream=io.StringIO())
    c = out["trainer"].cfg
    assert (c.sd_ratio, c.recent_window, c.recent_window_layers, c.postprocessor, c.input_dropout) == (0.5, 8, 1, "l2", 0.0)
    assert c.tasks == (("listen_plus", 1, "binary"), ("like", 2, "binary")) and all(l == l for l in out["losses"])
    assert any("'bogus'" in str(x.message) for x in w)


def test_event_store_feeds_the_eleven_table_feature_set(tmp_path):
    """Event store + ``embedding.tables: yambda``: every batch carries the keyed jagged features (item / artist / album per
    token from the store's item maps, user id and hashed crosses per sample) and the loop trains and evaluates on them."""
    import numpy as np
    from mlperf_training_b200.data.yambda import write_synthetic_event_store
    from mlperf_training_b200.trainer.hstu import run
    root = tmp_path / "store"
    write_synthetic_event_store(str(root), 80, 60, 3000, days=3, seed=2)
    rng = np.random.default_rng(0)
    np.save(root / "item_artist.npy", rng.integers(0, 500, size=3000))
    np.save(root / "item_album.npy", rng.integers(0, 900, size=3000))
    e = _exp(train_steps=4, eval_interval_steps=2, num_eval_batches=1, batch_per_gpu=4,
             embedding=dict(dim=16, tables="yambda", table_scale=2000), data=dict(kind="yambda", path=str(root), min_history=4, max_history=30))
    out = run(e, device="cpu", stream=io.StringIO())
    assert len(out["losses"]) >= 3 and all(l == l for l in out["losses"])
    tr = out["trainer"]
    b = tr.data.batch_at(0, 0)
    uih, cand = b["samples"].uih, b["samples"].candidates
    rows = {t.name: t.rows for t in tr.table.configs}
    art, alb = torch.from_numpy(np.load(root / "item_artist.npy")), torch.from_numpy(np.load(root / "item_album.npy"))
    hist = ~torch.isin(torch.arange(b["total"]), b["offsets"][1:].long() - 1)            # one candidate per sample: its last event
    raw = b["item_ids"]
    assert torch.equal(uih["uih_item_id"][0], raw[hist] % rows["item_id"]) and torch.equal(cand["item_id"][0], raw[~hist] % rows["item_id"])
    assert torch.equal(uih["uih_artist_id"][0], art[raw[hist]] % rows["artist_id"]) and torch.equal(cand["album_id"][0], alb[raw[~hist]] % rows["album_id"])
    assert torch.equal(uih["uid"][0], b["users"] % rows["uid"]) and all(int(uih[f"cross_{k}"][0].max()) < rows[f"cross_{k}"] for k in range(7))


def test_preprocessed_sessions_convert_to_an_event_store(tmp_path):
    """``train_sessions.parquet`` (list columns per session) and the item -> artist / album parquets become an event store
    whose samples carry the listen-plus label and the item maps."""
    import numpy as np
    import pandas as pd
    from mlperf_training_b200.data import prep
    from mlperf_training_b200.data.yambda import EventStoreDataset
    rng = np.random.default_rng(0)
    rows = []
    for uid in range(12):
        t = 1_600_000_000
        for sess in range(3):
            n = int(rng.integers(4, 9))
            ts = t + np.cumsum(rng.integers(1, 300, size=n))
            t = int(ts[-1]) + 4000
            rows.append({"uid": uid, "session_id": sess, "item_ids": rng.integers(0, 50, size=n).tolist(), "timestamps": ts.tolist(),
                         "event_types": rng.choice([0, 0, 0, 1, 2], size=n).tolist(), "is_organic": [1] * n,
                         "played_ratio_pct": rng.choice([10.0, 49.0, 50.0, 100.0, np.nan], size=n).tolist()})
    proc, meta = tmp_path / "processed", tmp_path / "meta"
    proc.mkdir(), meta.mkdir()
    pd.DataFrame(rows).sample(frac=1.0, random_state=1).to_parquet(proc / "train_sessions.parquet")     # rows in any order
    pd.DataFrame({"item_id": np.arange(50), "artist_id": np.arange(50) // 5}).to_parquet(meta / "artist_item_mapping.parquet")
    pd.DataFrame({"item_id": np.arange(50), "album_id": np.arange(50) // 2}).to_parquet(meta / "album_item_mapping.parquet")
    assert prep.main(["convert-events", str(proc), str(tmp_path / "store"), "--metadata-dir", str(meta)]) == 0
    ds = EventStoreDataset(str(tmp_path / "store"), 2, min_history=3, max_history=12, holdout=0.0)
    n_events = sum(len(r["item_ids"]) for r in rows)
    assert len(ds.item) == n_events and ds.item_artist.tolist() == (np.arange(50) // 5).tolist()
    user = np.asarray(ds.user)
    assert (np.diff(user) >= 0).all() and all((np.diff(np.asarray(ds.ts)[user == u]) >= 0).all() for u in range(12))
    # listen-plus: a listen played for at least half; likes and other events carry no played flag
    flat_kind = np.concatenate([np.asarray(r["event_types"]) for r in sorted(rows, key=lambda r: (r["uid"], r["session_id"]))])
    flat_ratio = np.nan_to_num(np.concatenate([np.asarray(r["played_ratio_pct"], dtype=np.float32)
                                               for r in sorted(rows, key=lambda r: (r["uid"], r["session_id"]))]))
    assert np.array_equal(np.asarray(ds.kind), flat_kind) and np.array_equal(np.asarray(ds.played), ((flat_kind == 0) & (flat_ratio >= 50)).astype(np.uint8))
    b = ds.batch_at(0)
    assert b["item_ids"].numel() == b["total"] and set(b["users"].tolist()) <= set(range(12))
