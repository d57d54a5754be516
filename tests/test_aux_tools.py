"""Auxiliary tools: trace repair and step-wall report, the stdout filter, dataset staging with its
sentinel, and the GPU idle check against a fake ``nvidia-smi``."""
import json
import os
import stat
import subprocess
import sys

from mlperf_training_b200.utils.profiler import clean_trace, gpu_peak_tflops, step_wall_report

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_trace_repair_and_step_report(tmp_path):
    ev = [
        {"ph": "X", "cat": "user_annotation", "name": "train_step#0", "ts": 100, "dur": 100, "pid": 1, "tid": 1},
        {"ph": "X", "cat": "kernel", "name": "warmup", "ts": 10, "dur": 5, "pid": 0, "tid": 7},
        {"ph": "X", "cat": "kernel", "name": "a", "ts": 110, "dur": 30, "pid": 0, "tid": 7},
        {"ph": "X", "cat": "kernel", "name": "b", "ts": 130, "dur": 30, "pid": 0, "tid": 7},      # overlaps a on its lane
        {"ph": "X", "cat": "kernel", "name": "c", "ts": 190, "dur": -3, "pid": 0, "tid": 7},      # negative duration
        {"ph": "M", "name": "process_name", "pid": 0},
    ]
    p = tmp_path / "trace.json"
    p.write_text(json.dumps({"traceEvents": ev}))
    stats = clean_trace(p, trim_before_us=50)
    assert stats == {"dropped": 1, "clipped": 1, "deoverlapped": 1}
    out = json.loads(p.read_text())["traceEvents"]
    b = next(e for e in out if e.get("name") == "b")
    assert b["ts"] == 140 and b["dur"] == 20 and all(e.get("name") != "warmup" for e in out)
    rep = step_wall_report(p)
    assert rep["steps"] == [{"wall_us": 100, "gpu_busy_us": 50}]
    assert gpu_peak_tflops("NVIDIA B200") == 2250.0


def test_stdout_filter_passes_only_mllog(tmp_path):
    code = (
        "import sys; sys.path.insert(0, %r)\n"
        "from mlperf_training_b200.mllog import suppress\n"
        "suppress.install(side_file=%r)\n"
        "print('noise line'); print(':::MLLOG {\"key\": \"x\"}'); print('RESULT,bench,,1,B200,now')\n"
        "import os; os.write(2, b'stderr noise\\n')\n"
        "suppress.restore(); print('after restore')\n"
    ) % (ROOT, str(tmp_path / "side.log"))
    env = {k: v for k, v in os.environ.items() if k != "B200_VERBOSE"}
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=120)
    assert r.returncode == 0, r.stderr
    lines = r.stdout.splitlines()
    assert ':::MLLOG {"key": "x"}' in lines and "RESULT,bench,,1,B200,now" in lines and "after restore" in lines
    assert "noise line" not in lines and "stderr noise" not in r.stderr
    assert "noise line" in (tmp_path / "side.log").read_text()


def test_stage_dataset_sentinel(tmp_path):
    src, dst = tmp_path / "src", tmp_path / "dst"
    src.mkdir()
    (src / "a.bin").write_bytes(b"x" * 1000)
    script = os.path.join(ROOT, "workloads", "common", "stage_dataset_local.sh")
    r1 = subprocess.run(["bash", script, str(src), str(dst)], capture_output=True, text=True, timeout=60)
    assert r1.returncode == 0 and (dst / "a.bin").exists()
    assert (dst / ".stage_complete").read_text().splitlines()[0] == str(src)
    r2 = subprocess.run(["bash", script, str(src), str(dst)], capture_output=True, text=True, timeout=60)
    assert "already staged" in r2.stdout


def test_gpu_idle_check_with_fake_nvidia_smi(tmp_path):
    fake = tmp_path / "nvidia-smi"
    script = os.path.join(ROOT, "workloads", "common", "check_gpus_idle.sh")

    def run(mem_lines, apps):
        fake.write_text("#!/bin/bash\ncase \"$*\" in *compute-apps*) printf '%s' \"" + apps + "\";; *) printf '" + mem_lines + "';; esac\n")
        fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
        env = dict(os.environ, PATH=f"{tmp_path}:{os.environ['PATH']}")
        return subprocess.run(["bash", script], capture_output=True, text=True, env=env, timeout=60)

    assert run("0, 3\\n1, 0\\n", "").returncode == 0
    busy = run("0, 3\\n1, 40960\\n", "")
    assert busy.returncode == 1 and "GPU 1" in busy.stdout
    assert run("0, 0\\n", "4242\\n").returncode == 1


def test_model_fingerprint_tracks_the_initial_weights(capsys, monkeypatch):
    import io
    import torch
    from mlperf_training_b200.models.gpt import GPT, GPTConfig
    from mlperf_training_b200.utils.metrics import model_fingerprint
    cfg = GPTConfig(n_layers=1, hidden=32, n_heads=2, n_kv_heads=1, head_dim=16, ffn_hidden=64, vocab_size=64, seq_len=8, dtype="fp32")
    a, rows = model_fingerprint(GPT(cfg, seed=3))
    b, _ = model_fingerprint(GPT(cfg, seed=3))
    c, _ = model_fingerprint(GPT(cfg, seed=4))
    assert a == b and a != c and len(a) == 64
    assert rows == sorted(rows) and all(n > 0 for _, n, _, _ in rows)
    m = GPT(cfg, seed=3)
    with torch.no_grad():
        next(m.parameters()).view(-1)[0] += 1e-3
    assert model_fingerprint(m)[0] != a                                     # one changed element changes the digest
    monkeypatch.setenv("INIT_CHECKSUM", "1")
    from mlperf_training_b200.trainer.loop import run
    run(dict(model=cfg.to_dict(), global_batch=2, micro_batch=1, train_iters=1, warmup_train_steps=0), device="cpu", stream=io.StringIO())
    assert "[init] model fingerprint " in capsys.readouterr().out


def test_mxfp8_site_probe_reports_snr_and_is_scale_invariant():
    import math
    import torch
    from mlperf_training_b200.utils.numerics import cosine, linear_site_report, main, snr_db
    g = torch.Generator().manual_seed(0)
    x, w, dy = torch.randn(256, 384, generator=g), torch.randn(128, 384, generator=g) * 0.02, torch.randn(256, 128, generator=g) * 1e-3
    assert snr_db(x, x) == math.inf and abs(cosine(x, 2 * x) - 1.0) < 1e-12
    assert abs(snr_db(x, x * 1.1) - 20.0) < 1e-3                                     # 10 % error -> 20 dB
    rep = linear_site_report(x, w, dy)
    assert set(rep) == {"fwd", "dgrad", "wgrad"}
    for site in rep.values():                                                       # e4m3 + per-32 scales: about 30 dB per GEMM
        assert 22.0 < site["snr_db"] < 45.0 and site["cosine"] > 0.995
    # power-of-two rescaling of an operand moves only the block exponents
    rep2 = linear_site_report(x * 1024, w / 64, dy * 4)
    for k in rep:
        assert abs(rep2[k]["snr_db"] - rep[k]["snr_db"]) < 0.05
    assert main(["--tokens", "128", "--in", "128", "--out", "128", "--outliers", "0.01"]) == 0
    # through the training path: the narrower the elements, the lower the ratio; the bare-operand probe agrees for mxfp8
    from mlperf_training_b200.utils.numerics import recipe_report
    torch.manual_seed(0)
    by = {p: recipe_report(x, w, dy, p) for p in ("mxfp8", "mxfp6", "mxfp4", "fp8")}
    assert all(abs(by["mxfp8"][k]["snr_db"] - rep[k]["snr_db"]) < 1.0 for k in rep)
    assert by["mxfp8"]["fwd"]["snr_db"] > by["mxfp6"]["fwd"]["snr_db"] > by["mxfp4"]["fwd"]["snr_db"] > 10.0
    assert by["fp8"]["fwd"]["snr_db"] > 22.0 and by["mxfp4"]["wgrad"]["cosine"] > 0.95
    assert main(["--tokens", "128", "--in", "128", "--out", "128", "--precision", "a6w4"]) == 0


def test_startup_timeline_phases():
    from mlperf_training_b200.utils.metrics import StartupTimeline
    ticks = iter([0.0, 1.5, 4.0])
    t = StartupTimeline(clock=lambda: next(ticks))
    assert t.mark("model") == 1.5 and t.mark("warmup") == 2.5
    assert t.report() == {"phases": {"model": 1.5, "warmup": 2.5}, "total_s": 4.0}


def test_startup_selfcheck_runs_and_fails_closed(monkeypatch):
    from mlperf_training_b200.ops import kernels as K
    from mlperf_training_b200.ops import selfcheck
    rep = selfcheck.run_selfcheck("cpu")
    assert set(rep) >= {"gemm", "block-scaled gemm", "attention", "cross entropy"} and max(rep.values()) == 0.0
    assert selfcheck.main(["--device", "cpu"]) == 0
    # a kernel that disagrees with its oracle stops the run
    real = K.swiglu_fwd
    calls = {"n": 0}

    def broken(gu):
        calls["n"] += 1
        out = real(gu)
        return out * 1.5 if calls["n"] % 2 == 1 else out           # the "device" side is off by 50 %
    monkeypatch.setattr(K, "swiglu_fwd", broken)
    import pytest
    with pytest.raises(RuntimeError, match="swiglu"):
        selfcheck.run_selfcheck("cpu")
