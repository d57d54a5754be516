"""Event-store dataset (anchors, three-pool history, windows, deterministic split and rank slices),
allocator growth monitor, performance line."""
import json

import numpy as np

from mlperf_training_b200.data.yambda import EventStoreDataset, write_event_store
from mlperf_training_b200.utils.alloc import GrowthMonitor, pregrow, recommended_env
from mlperf_training_b200.utils.metrics import PerfLogger


def _store(tmp_path, users=40, events=120, seed=0):
    rng = np.random.default_rng(seed)
    user = np.repeat(np.arange(users), events)
    ts = 1_600_000_000 + rng.integers(0, 5 * 86_400, size=users * events)
    item = rng.integers(0, 500, size=users * events)
    kind = rng.choice([0, 0, 0, 1, 2], size=users * events).astype(np.uint8)
    write_event_store(str(tmp_path / "store"), user, item, ts, kind, played=rng.integers(0, 2, size=users * events))
    return str(tmp_path / "store")


def test_event_store_batches(tmp_path):
    root = _store(tmp_path)
    ds = EventStoreDataset(root, batch=4, max_history=30, min_history=8, holdout=0.2, salt=3)
    ev = EventStoreDataset(root, batch=4, max_history=30, min_history=8, holdout=0.2, salt=3, split="eval")
    tr_users, ev_users = set(ds.user[ds.anchors].tolist()), set(ev.user[ev.anchors].tolist())
    assert tr_users and ev_users and not (tr_users & ev_users)                      # the split is by user
    assert ds.num_windows >= 4
    a0, a1 = ds.window_anchors(1, 0, 2), ds.window_anchors(1, 1, 2)
    assert not set(a0.tolist()) & set(a1.tolist())                                  # rank slices are disjoint
    assert np.all(np.diff(np.asarray(ds.ts)[a0]) >= 0)                              # time order inside a window
    b = ds.batch_at(0)
    assert b["offsets"].tolist()[0] == 0 and b["total"] == int(b["offsets"][-1]) and b["rows"] % 128 == 0
    lens = b["lengths"].tolist()
    assert all(9 <= n <= 31 for n in lens)                                          # >= min_history + target, <= cap + target
    for i in range(4):                                                              # per user: time-ordered, target last
        seg = b["timestamps"][b["offsets"][i]:b["offsets"][i + 1]]
        assert bool((seg[1:] >= seg[:-1]).all())
    again = EventStoreDataset(root, batch=4, max_history=30, min_history=8, holdout=0.2, salt=3).batch_at(0)
    assert again["item_ids"].tolist() == b["item_ids"].tolist()                     # exact-once resume contract
    n_steps = sum(ds.batches_in_window(w) for w in range(ds.num_windows))
    assert ds.batch_at(n_steps - 1)["total"] > 0


def test_growth_monitor_and_perf_line(tmp_path):
    state = {"reserved_bytes.all.current": 100, "segment.all.allocated": 2, "num_alloc_retries": 0}
    mon = GrowthMonitor(stats=lambda: dict(state))
    assert mon.check(1) is None and "no growth" in mon.report()
    state["reserved_bytes.all.current"] = 100 + (3 << 20)
    ev = mon.check(2)
    assert ev["step"] == 2 and ev["reserved"] == 3 << 20 and "3.0 MiB" in mon.report()
    assert pregrow(1 << 20) >= 0 and "expandable_segments" in recommended_env()["PYTORCH_CUDA_ALLOC_CONF"]
    p = PerfLogger(flops_per_sample=1e12, world=2, peak_tflops=1000.0, jsonl=str(tmp_path / "m.jsonl"))
    p.step(8)
    p.pause(), p.resume()
    rec = p.line(1, {"loss": 0.5})
    assert rec["samples_per_s"] > 0 and abs(rec["mfu"] - rec["tflops_algo_per_gpu"] / 1000.0) < 1e-12
    assert json.loads((tmp_path / "m.jsonl").read_text().splitlines()[0])["loss"] == 0.5


def test_hstu_run_on_event_store_with_warmup(tmp_path):
    import io
    from mlperf_training_b200.mllog import check_compliance
    from mlperf_training_b200.trainer.hstu import run
    root = _store(tmp_path, users=60, events=100)
    exp = dict(batch_per_gpu=4, train_steps=6, warmup_steps=2, eval_interval_steps=3, num_eval_batches=1,
               model=dict(layers=1, dim=32, heads=2, d_qk=16, d_v=16, max_seq_len=48, dtype="fp32", mlp_hidden=16,
                          num_positions=64, num_time_buckets=32),
               embedding=dict(rows=500, dim=16),
               data=dict(kind="yambda", root=root, max_history=30, min_history=8, holdout=0.3, salt=1), cold_prefetch_steps=2)
    out = run(exp, device="cpu", stream=io.StringIO())
    assert out["trainer"].data.readahead == 2
    assert len(out["losses"]) == 6 and all(l == l for l in out["losses"]) and len(out["aucs"]) == 2
    assert check_compliance(out["records"]) == []
    # warm-up left no trace: a run without it starts from the same state
    ref = run(dict(exp, warmup_steps=0), device="cpu", stream=io.StringIO())
    assert abs(ref["losses"][0] - out["losses"][0]) < 1e-6


def test_energy_monitor_integrates_power():
    import time
    from mlperf_training_b200.utils.energy import EnergyMonitor
    m = EnergyMonitor(interval_s=0.05, reader=lambda: [100.0, 50.0]).start()
    time.sleep(0.4)
    rep = m.stop()
    assert rep["samples"] >= 3 and rep["peak_w"] == 150.0
    assert 150.0 * 0.15 < rep["energy_j"] < 150.0 * 0.6


def test_replica_checksum_single_process():
    import torch
    from mlperf_training_b200.models.gpt import GPT, GPTConfig
    from mlperf_training_b200.parallel.engine import OptimConfig, ZeroEngine
    m = GPT(GPTConfig(n_layers=1, hidden=32, n_heads=2, n_kv_heads=1, head_dim=16, ffn_hidden=64, vocab_size=64, seq_len=8,
                      dtype="fp32"), seed=0)
    assert ZeroEngine(m, OptimConfig()).replica_checksum_spread() == 0.0


def test_sequence_file_dataset_semantics(tmp_path):
    import csv
    import numpy as np
    from mlperf_training_b200.data.sequences import (SequenceFileDataset, parse_sequence, split_history_candidates,
                                                      write_synthetic_sequences)
    assert parse_sequence("3,5,9") == [3, 5, 9] and parse_sequence("[1, 2]") == [1, 2] and parse_sequence(7) == [7]
    assert split_history_candidates([1, 2, 3, 4, 5], 2) == ([1, 2, 3], [4, 5])
    path = tmp_path / "ml.csv"
    with open(path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["user_id", "sequence_item_ids", "sequence_ratings", "sequence_timestamps"])
        w.writerow([0, "10,11,12,13,14,15", "1,3,5,4.5,2,4", "100,200,300,400,500,600"])
        w.writerow([1, "20,21", "5,1", "7,8"])                       # not longer than the candidates: skipped
        w.writerow([2, "[30, 31, 32]", "[5.0, 2.0, 3.5]", "[5, 9, 50]"])
    ds = SequenceFileDataset(str(path), batch=2, num_candidates=2, max_history=3, action_weights=(1, 1, 2, 4, 4), label_bit=8)
    assert len(ds) == 2
    b = ds.build_batch(np.array([0, 1]))
    assert b["offsets"].tolist() == [0, 5, 8] and b["num_targets"].tolist() == [2, 2] and b["total"] == 8 and b["rows"] == 128
    # user 0: history 10..13 cut to its first 3 events, candidates 14, 15 (ratings 2 -> 0, 4 -> label bit)
    assert b["item_ids"][:5].tolist() == [10, 11, 12, 14, 15]
    assert b["actions"][:5].tolist() == [1, 2, 4, 0, 8]
    assert b["timestamps"][:5].tolist() == [100, 200, 300, 300, 300]                 # candidates carry the query time
    assert b["item_ids"][5:].tolist() == [30, 31, 32] and b["actions"][5:].tolist() == [4, 0, 8]
    # KuaiRand layout: stored masks, the label is one of their bits
    kpath = tmp_path / "kr.csv"
    with open(kpath, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["user_id", "video_id", "action_weights", "time_ms"])
        w.writerow([5, "1,2,3,4", "6,1,3,5", "10,20,30,40"])
    kd = SequenceFileDataset(str(kpath), batch=1, kind="kuairand", num_candidates=1, label_bit=1)
    kb = kd.build_batch(np.array([0]))
    assert kb["actions"].tolist() == [6, 1, 3, 1] and kb["timestamps"].tolist() == [10, 20, 30, 30]
    # synthetic file: disjoint train / eval users, deterministic per-rank slices that tile a step
    spath = tmp_path / "syn.csv"
    write_synthetic_sequences(str(spath), users=200, items=500, seed=3)
    tr = SequenceFileDataset(str(spath), batch=4, split="train", eval_fraction=0.25)
    ev = SequenceFileDataset(str(spath), batch=4, split="eval", eval_fraction=0.25)
    assert len(tr) + len(ev) == 200 and 20 < len(ev) < 80
    a0, a1 = tr.batch_at(3, 0, world=2), tr.batch_at(3, 1, world=2)
    again = tr.batch_at(3, 0, world=2)
    assert a0["item_ids"].tolist() == again["item_ids"].tolist()
    assert a0["item_ids"].tolist() != a1["item_ids"].tolist()
    per = tr.steps_per_pass(2)
    assert tr.batch_at(per + 3, 0, world=2)["item_ids"].tolist() != a0["item_ids"].tolist()      # the next pass is reshuffled


def test_hstu_run_on_sequence_file(tmp_path):
    import io
    from mlperf_training_b200.data.sequences import write_synthetic_sequences
    from mlperf_training_b200.trainer.hstu import run
    path = tmp_path / "ml.csv"
    write_synthetic_sequences(str(path), users=120, items=400, min_len=6, max_len=40, seed=1)
    exp = dict(batch_per_gpu=4, train_steps=5, warmup_steps=1, eval_interval_steps=5, num_eval_batches=1,
               model=dict(layers=1, dim=32, heads=2, d_qk=16, d_v=16, max_seq_len=48, dtype="fp32", mlp_hidden=16,
                          num_positions=64, num_time_buckets=32),
               embedding=dict(rows=500, dim=16),
               data=dict(kind="sequences", path=str(path), format="movielens", num_candidates=2, max_history=30, eval_fraction=0.3))
    out = run(exp, device="cpu", stream=io.StringIO())
    assert len(out["losses"]) == 5 and all(l == l for l in out["losses"]) and len(out["aucs"]) == 1


def test_prep_cli_writes_synthetic_hstu_data(tmp_path):
    from mlperf_training_b200.data.prep import main
    from mlperf_training_b200.data.sequences import SequenceFileDataset
    assert main(["synthetic-events", str(tmp_path / "store"), "--users", "50", "--events-per-user", "80", "--items", "300", "--days", "4"]) == 0
    ds = EventStoreDataset(str(tmp_path / "store"), batch=4, max_history=30, min_history=8, holdout=0.2, salt=3)
    assert ds.num_windows >= 3 and ds.batch_at(0)["total"] > 0
    items = np.asarray(ds.item)
    assert np.bincount(items).max() > 5 * max(np.median(np.bincount(items)), 1)       # a popular head
    assert main(["synthetic-sequences", str(tmp_path / "kr.csv"), "--users", "30", "--items", "200", "--kind", "kuairand", "--max-len", "20"]) == 0
    assert len(SequenceFileDataset(str(tmp_path / "kr.csv"), batch=2, kind="kuairand")) == 30


def test_window_boundaries_are_announced(tmp_path, monkeypatch, capsys):
    import io
    from mlperf_training_b200.trainer.hstu import run
    root = _store(tmp_path, users=60, events=100)
    ds = EventStoreDataset(root, batch=4, max_history=30, min_history=8, holdout=0.3, salt=1)
    per = [ds.batches_in_window(w) for w in range(ds.num_windows)]
    assert [ds.window_of_step(s) for s in (0, per[0] - 1, per[0])] == [0, 0, 1] if per[0] > 1 else True
    monkeypatch.setenv("WINDOW_BARRIER_DEBUG", "1")
    steps = per[0] + 2
    run(dict(batch_per_gpu=4, train_steps=steps, eval_interval_steps=0,
             model=dict(layers=1, dim=32, heads=2, d_qk=16, d_v=16, max_seq_len=48, dtype="fp32", mlp_hidden=16,
                        num_positions=64, num_time_buckets=32),
             embedding=dict(rows=500, dim=16), data=dict(kind="yambda", root=root, max_history=30, min_history=8, holdout=0.3, salt=1)),
        device="cpu", stream=io.StringIO())
    lines = [l for l in capsys.readouterr().out.splitlines() if l.startswith("[window-barrier]")]
    assert len(lines) == 2 and "window 0" in lines[0] and "window 1" in lines[1]


def test_event_store_read_ahead_covers_the_batches(tmp_path):
    root = _store(tmp_path, users=40, events=120)
    ds = EventStoreDataset(root, batch=4, max_history=30, min_history=8, holdout=0.2, salt=3)
    for step in (0, 1, 5):
        anchors = ds.step_anchors(step, 1, 2)
        b = ds.batch_at(step, 1, world=2)
        # the batch's last event of every sample is its anchor
        ends = (b["offsets"][1:] - 1).tolist()
        assert b["item_ids"][ends].tolist() == np.asarray(ds.item)[anchors].tolist()
    ranges = ds.event_ranges([0, 1], 0, 1)
    assert all(lo < hi for lo, hi in ranges) and all(a[1] < b[0] for a, b in zip(ranges, ranges[1:]))      # merged, disjoint
    covered = np.zeros(len(ds.user), bool)
    for lo, hi in ranges:
        covered[lo:hi] = True
    for step in (0, 1):
        for a in ds.step_anchors(step):
            assert covered[ds._history(int(a))].all() and covered[a]
    n = ds.prefetch([0, 1])
    width = sum(arr.dtype.itemsize for arr in (ds.item, ds.ts, ds.kind, ds.played))
    assert n == sum(hi - lo for lo, hi in ranges) * width
