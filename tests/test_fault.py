"""Failure detection without a GPU fault: a rank that stops heart-beating is noticed by the others
between steps; a collective whose peer never joins ends through the process-group timeout; the
straggler detector and timed barrier on one process."""
import io
import os
import subprocess
import sys

from mlperf_training_b200.parallel import health

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "multi", "fault_worker.py")


def test_silent_rank_is_detected_through_heartbeats(tmp_path):
    store = str(tmp_path / "store")
    procs = [subprocess.Popen([sys.executable, WORKER, "heartbeat", store, str(r), "3"], stdout=subprocess.PIPE,
                              stderr=subprocess.PIPE, text=True) for r in range(3)]
    outs = [p.communicate(timeout=120) for p in procs]
    assert procs[1].returncode == 0
    for r in (0, 2):
        assert procs[r].returncode == health.EXIT_RANK_FAILURE, outs[r]
        assert "detected [1]" in outs[r][0]


def test_collective_with_missing_peer_times_out(tmp_path):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29661", WORKER, "timeout"],
                       env=env, capture_output=True, text=True, timeout=180)
    assert "rank 0 collective ended with" in r.stdout, r.stdout[-1500:] + r.stderr[-1500:]


def test_straggler_detector_and_timed_barrier():
    d = health.StragglerDetector(interval=3, factor=1.5)
    assert d.record(0.1) is None and d.record(0.1) is None
    rep = d.record(0.1)
    assert rep["stragglers"] == [] and abs(rep["median"] - 0.1) < 1e-9
    buf = io.StringIO()
    assert health.timed_barrier(warn_after_s=0.0, out=buf) >= 0.0
    assert health.pg_timeout(7).total_seconds() in (7.0, float(os.environ.get("PG_TIMEOUT_S", 7)))


def test_supervisor_decisions():
    import io
    import json
    from mlperf_training_b200.trainer.supervisor import EXIT_INJECTED, EXIT_RANK_FAILURE, decide, next_world, supervise, worst_rank_code
    assert next_world(8, 8, 2) == 4 and next_world(4, 8, 2) == 2 and next_world(2, 8, 2) is None and next_world(6, 6, 1) == 3
    assert decide(0, 0, 3, 8, 8, 1, False) == ("done", 8)
    assert decide(EXIT_INJECTED, 0, 3, 8, 8, 2, True) == ("restart", 8)            # a crash after a save: same size again
    assert decide(EXIT_RANK_FAILURE, 1, 3, 8, 8, 2, True) == ("restart", 4)        # a lost rank: next smaller divisor
    assert decide(EXIT_RANK_FAILURE, 1, 3, 2, 8, 2, True) == ("give_up", 2)
    assert decide(1, 3, 3, 8, 8, 1, False) == ("give_up", 8)
    assert worst_rank_code(1, "failed (exitcode: 43) local_rank: 1") == EXIT_RANK_FAILURE and worst_rank_code(1, "boom") == 1
    # a scripted job: loses a rank, shrinks, is hit by an injected crash, then finishes
    script = iter([EXIT_RANK_FAILURE, EXIT_INJECTED, 0])
    seen = []

    def fake(world, args):
        seen.append(world)
        return next(script)
    out = io.StringIO()
    assert supervise(8, ["pretrain"], max_restarts=3, shrink=True, min_world=2, out=out, run=fake) == 0
    assert seen == [8, 4, 4]
    lines = [json.loads(l) for l in out.getvalue().splitlines()]
    assert [l["action"] for l in lines] == ["restart", "restart", "done"] and lines[0]["next_world"] == 4
    # out of restarts
    assert supervise(2, [], max_restarts=1, run=lambda w, a: 7, out=io.StringIO()) == 7


def test_supervisor_relaunches_after_injected_crash_gloo(tmp_path):
    import json
    yaml = tmp_path / "exp.yaml"
    yaml.write_text(f"""
modules:
  pre_trainer:
    framework: b200
    overrides:
      global_batch: 4
      micro_batch: 1
      train_iters: 4
      warmup_train_steps: 0
      die_at_step: 2
      checkpoint_dir: {tmp_path / 'ck'}
      mllog_file: {tmp_path / 'ml.log'}
      model: {{n_layers: 1, hidden: 32, n_heads: 2, n_kv_heads: 1, head_dim: 16, ffn_hidden: 64, vocab_size: 64, seq_len: 16, dtype: fp32}}
      data: {{kind: synthetic}}
""")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT, B200_QUIET="0")
    r = subprocess.run([sys.executable, "-m", "mlperf_training_b200.trainer.supervisor", "--nproc", "2", "--max-restarts", "2", "--",
                        "pretrain", "--config", str(yaml), "--device", "cpu"], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    sup = [json.loads(l) for l in r.stdout.splitlines() if l.startswith('{"supervisor"')]
    assert [s["action"] for s in sup] == ["restart", "done"] and sup[0]["exit_code"] == 42 and sup[1]["exit_code"] == 0
    log = (tmp_path / "ml.log").read_text()
    assert log.count("run_start") == 1 and log.count("run_stop") == 1                 # one run, resumed in place


def test_lost_rank_is_noticed_then_run_shrinks_and_resumes_gloo(tmp_path):
    """The whole chain on CPU ranks: a rank leaves silently between steps, the others notice at the
    host-side rendezvous before the next step and exit 43, the supervisor relaunches on half the
    ranks, and the run resumes from the last checkpoint with its optimizer state re-cut."""
    import json
    yaml = tmp_path / "exp.yaml"
    yaml.write_text(f"""
modules:
  pre_trainer:
    framework: b200
    overrides:
      global_batch: 4
      micro_batch: 1
      train_iters: 5
      warmup_train_steps: 0
      checkpoint_every: 2
      checkpoint_dir: {tmp_path / 'ck'}
      mllog_file: {tmp_path / 'ml.log'}
      heartbeat_timeout_s: 3
      vanish_at_step: 3
      vanish_rank: 1
      model: {{n_layers: 1, hidden: 32, n_heads: 2, n_kv_heads: 1, head_dim: 16, ffn_hidden: 64, vocab_size: 64, seq_len: 16, dtype: fp32}}
      data: {{kind: synthetic}}
""")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT, B200_QUIET="0")
    r = subprocess.run([sys.executable, "-m", "mlperf_training_b200.trainer.supervisor", "--nproc", "4", "--max-restarts", "2", "--shrink",
                        "--min-nproc", "2", "--", "pretrain", "--config", str(yaml), "--device", "cpu"],
                       env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    sup = [json.loads(l) for l in r.stdout.splitlines() if l.startswith('{"supervisor"')]
    assert [(s["world"], s["exit_code"], s["action"]) for s in sup] == [(4, 43, "restart"), (2, 0, "done")], sup
    assert "rank failure detected" in r.stdout + r.stderr
    log = (tmp_path / "ml.log").read_text()
    assert log.count("run_start") == 1 and log.count("run_stop") == 1
