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
