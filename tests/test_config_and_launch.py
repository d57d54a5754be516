"""Config system, MLLOG stream and the single-box launch surface (CPU)."""
import io
import os
import subprocess
import sys
from pathlib import Path

import pytest

from mlperf_training_b200.config import loader
from mlperf_training_b200.mllog import MLLogger, ThroughputTimer, check_compliance, parse_log

REPO = Path(__file__).resolve().parent.parent


def test_env_helpers():
    env = {"A": "3", "B": "0", "C": "x:1,y:2", "D": ""}
    assert loader.env_int("A", 1, env) == 3 and loader.env_int("Z", 7, env) == 7 and loader.env_int("D", 5, env) == 5
    assert loader.env_bool("B", True, env) is False and loader.env_bool("A", False, env) is True
    assert loader.env_str_map("C", "", env) == {"x": "1", "y": "2"}
    assert loader.env_float("A", 0.0, env) == 3.0


def test_shell_defaults_env_wins(tmp_path):
    f = tmp_path / "config_X.sh"
    f.write_text('# comment\nexport GBS=32\nexport LR=8e-4 # trailing\nexport NAME="a b"\nexport DER=${GBS}_x\nif true; then :; fi\n')
    env = {"GBS": "4"}
    applied = loader.load_shell_defaults(f, env)
    assert env["GBS"] == "4" and "GBS" not in applied
    assert env["LR"] == "8e-4" and env["NAME"] == "a b" and env["DER"] == "4_x"


def test_yaml_substitution_and_layering(tmp_path):
    (tmp_path / "base.yaml").write_text("lr: 1.0e-3\nglobal_batch: 8\ndata:\n  kind: synthetic\n")
    (tmp_path / "m.yaml").write_text("preset: llama3.1-8b\n")
    (tmp_path / "exp.yaml").write_text(
        "name: ${NAME:demo}\nmodules:\n  pre_trainer:\n    config: base.yaml\n    model: m.yaml\n    overrides:\n"
        "      global_batch: ${GBS:32}\n      flag: ${FLAG:true}\n      model:\n        seq_len: ${SEQ:128}\n      text: run_${NAME:demo}\n")
    cfg = loader.load_experiment(tmp_path / "exp.yaml", env={"GBS": "16"}, overrides=["modules.pre_trainer.resolved.lr=0.5"])
    r = cfg["modules"]["pre_trainer"]["resolved"]
    assert r["global_batch"] == 16 and r["flag"] is True and r["lr"] == 0.5
    assert r["model"] == {"preset": "llama3.1-8b", "seq_len": 128} and r["text"] == "run_demo" and r["data"]["kind"] == "synthetic"
    with pytest.raises(KeyError):
        loader.substitute({"x": "${MISSING}"}, env={})


def test_shipped_experiments_resolve():
    for exp in REPO.glob("workloads/*/conf/*.yaml"):
        cfg = loader.load_experiment(exp, env={})
        mods = cfg["modules"]
        assert all("resolved" in m for m in mods.values()), exp


def test_mllog_lifecycle_and_compliance():
    buf = io.StringIO()
    t = [0.0]
    log = MLLogger(stream=buf, clock=lambda: t.__setitem__(0, t[0] + 1) or t[0])
    log.log_init_start()
    log.log_submission("llama31_8b")
    log.log_hyperparameters({"global_batch_size": 32, "junk": 1}, env={"MLLOG_SEED": "7"})
    log.log_init_stop_run_start()
    log.start("block_start")
    log.event("eval_accuracy", 3.4)
    log.end("block_stop")
    log.log_run_stop(True, samples=64, duration_s=2.0)
    recs = parse_log(buf.getvalue())
    assert [r["key"] for r in recs][:2] == ["cache_clear", "init_start"]
    assert {"seed", "global_batch_size"} <= {r["key"] for r in recs} and "junk" not in {r["key"] for r in recs}
    assert check_compliance(recs) == []
    assert any(r["key"] == "overall_throughput" and r["value"] == 32 for r in recs)
    assert "missing run_stop" in check_compliance(recs[:-3])


def test_throughput_timer_counts_only_step_time():
    t = [0.0]
    tm = ThroughputTimer(8, clock=lambda: t[0])
    for _ in range(3):
        tm.step_start(); t[0] += 2.0; tm.step_stop(); t[0] += 100.0  # eval / checkpoint time in between
    assert tm.samples == 24 and tm.throughput() == 4.0


def test_non_rank0_is_silent_but_syncs():
    calls = []
    buf = io.StringIO()
    log = MLLogger(rank=1, stream=buf, sync=lambda: calls.append(1))
    log.log_init_stop_run_start()
    assert buf.getvalue() == "" and len(calls) == 2


def test_run_and_time_end_to_end(tmp_path):
    """The launch surface on CPU: run_and_time.sh -> trainer CLI -> RESULT line + compliant MLLOG."""
    exp = REPO / "workloads" / "llama31_8b" / "conf" / "_test_tiny.yaml"
    exp.write_text(
        "modules:\n  pre_trainer:\n    config: pre_trainer.yaml\n    overrides:\n      benchmark: tiny\n      global_batch: 2\n"
        "      micro_batch: 1\n      train_iters: 3\n      eval_interval: 2\n      eval_iters: 1\n      warmup_train_steps: 1\n"
        "      model: {n_layers: 1, hidden: 32, n_heads: 2, n_kv_heads: 1, head_dim: 16, ffn_hidden: 64, vocab_size: 64, seq_len: 16, dtype: fp32}\n")
    try:
        env = dict(os.environ, WORKLOAD="llama31_8b", EXP="conf/_test_tiny.yaml", NGPU="1", CUDA_VISIBLE_DEVICES="",
                   PYTHONPATH=str(REPO))
        res = subprocess.run(["bash", str(REPO / "workloads/common/run_and_time.sh")], env=env, capture_output=True,
                             text=True, timeout=300)
        assert res.returncode == 0, res.stdout + res.stderr
        assert "STARTING TIMING RUN" in res.stdout and "RESULT,llama31_8b,," in res.stdout
        recs = parse_log(res.stdout)
        assert check_compliance(recs) == [] and any(r["key"] == "eval_accuracy" for r in recs)
        log = tmp_path / "trial.log"
        log.write_text(res.stdout)
        chk = subprocess.run([sys.executable, "-m", "mlperf_training_b200.mllog.compliance", str(log)], env=env,
                             capture_output=True, text=True)
        assert chk.returncode == 0 and "SUCCESS" in chk.stdout
    finally:
        exp.unlink()


def test_env_bootstrap_env_wins_and_partial_arm():
    from mlperf_training_b200.config.bootstrap import apply_env_bootstrap
    env = {"B_KEEP": "7"}
    bindings = {"a": "B_A", "keep": "B_KEEP", "x": "B_X", "y": "B_Y", "skip": "B_SKIP"}
    rep = apply_env_bootstrap(bindings, {"a": True, "keep": 3, "x": True, "y": False, "skip": None},
                              arms={"fp8_forward": ["x", "y"]}, environ=env)
    assert env["B_A"] == "1" and env["B_KEEP"] == "7" and env["B_Y"] == "0" and "B_SKIP" not in env
    assert rep.kept == {"B_KEEP": "7"} and rep.partial_arms == {"fp8_forward": {"on": ["x"], "off": ["y"]}}
    assert any("partial arm" in l for l in rep.lines())


def test_cli_takes_overrides_after_the_options(tmp_path, capsys):
    """``cli <mode> --config X --device cpu key=value ...``: the overrides may follow the options."""
    from mlperf_training_b200.trainer import cli
    exp = tmp_path / "tiny.yaml"
    exp.write_text(
        "modules:\n  pre_trainer:\n    overrides:\n      benchmark: tiny\n      global_batch: 2\n      micro_batch: 1\n"
        "      train_iters: 5\n      model: {n_layers: 1, hidden: 32, n_heads: 2, n_kv_heads: 1, head_dim: 16, ffn_hidden: 64, "
        "vocab_size: 64, seq_len: 16, dtype: fp32}\n")
    rc = cli.main(["pretrain", "--config", str(exp), "--device", "cpu", "modules.pre_trainer.resolved.train_iters=2"])
    out = capsys.readouterr().out
    assert rc == 0
    recs = parse_log(out)
    assert sum(r["key"] == "train_loss" for r in recs) == 2             # two iterations, not the file's five


_GPT_TINY = ["model.n_layers=2", "model.hidden=128", "model.n_heads=2", "model.n_kv_heads=2", "model.head_dim=64", "model.vocab_size=256",
             "model.seq_len=128", "model.dtype=fp32", "train_iters=2", "global_batch=2", "micro_batch=1", "eval_interval=0",
             "warmup_train_steps=0"]
_SHIPPED = {
    "workloads/llama31_8b/conf/llama3.1_8B-pretrain-mxfp8.yaml": ("pretrain", "pre_trainer", _GPT_TINY + ["model.ffn_hidden=256", "comm=nccl"]),
    "workloads/gpt_oss_20b/conf/gpt_oss_20B-mxfp8-pretrain.yaml": ("pretrain", "pre_trainer", _GPT_TINY + [
        "model.moe_ffn_hidden=128", "model.n_experts=4", "model.top_k=2", "model.window=64", "expert_parallel=1", "moe_dispatch=nccl"]),
    "workloads/gpt_oss_20b/conf/gpt_oss_20B-mxfp4-deosc-pretrain.yaml": ("pretrain", "pre_trainer", _GPT_TINY + [
        "model.moe_ffn_hidden=128", "model.n_experts=4", "model.top_k=2", "model.window=64", "expert_parallel=1", "moe_dispatch=nccl",
        "precision_schedule.deosc.start_step=0", "precision_schedule.deosc.period=2"]),
    "workloads/llama2_70b_lora/conf/llama2_70b_lora_posttrain.yaml": ("posttrain", "post_trainer", _GPT_TINY + ["model.ffn_hidden=256", "data.loss_last=32"]),
    "workloads/flux1/conf/flux.1_schnell_t2i-pretrain.yaml": ("flux", "flux_trainer", [
        "model.preset=tiny-mmdit", "model.img_size=64", "model.txt_tokens=16", "model.dtype=fp32", "train_iters=2", "global_batch=2",
        "local_batch=2", "warmup_train_steps=0", "warmup_eval_steps=0", "eval_every_samples=0", "fsdp.comm=nccl"]),
    "workloads/hstu/conf/hstu_yambda.yaml": ("hstu", "hstu_trainer", [
        "model.layers=1", "model.dim=64", "model.heads=2", "model.d_qk=32", "model.d_v=32", "model.max_seq_len=64", "model.dtype=fp32",
        "model.mlp_hidden=32", "model.num_positions=256", "model.num_time_buckets=64", "embedding.rows=300", "embedding.dim=32",
        "batch_per_gpu=4", "train_steps=2", "eval_interval_steps=0", "num_eval_batches=0", "data.length_median=12", "data.length_min=4",
        "data.length_max=40"]),
}


def test_every_shipped_experiment_file_is_covered():
    assert {str(p.relative_to(REPO)) for p in REPO.glob("workloads/*/conf/*.yaml")} == set(_SHIPPED)


@pytest.mark.parametrize("path", sorted(_SHIPPED))
def test_shipped_experiment_runs_through_the_cli_on_cpu(path, capsys):
    """Every shipped experiment file drives its trainer for two steps on CPU once the model is shrunk by overrides: the
    keys the file names are the keys the trainer reads."""
    from mlperf_training_b200.trainer import cli
    mode, module, over = _SHIPPED[path]
    rc = cli.main([mode, "--config", str(REPO / path), "--device", "cpu"] + [f"modules.{module}.resolved.{o}" for o in over])
    out = capsys.readouterr().out
    assert rc == 0 and "run_stop" in out


@pytest.mark.parametrize("kind", ["yambda", "sequences"])
def test_hstu_experiment_file_with_on_disk_data_kinds(kind, tmp_path, monkeypatch, capsys):
    """The shipped HSTU experiment file with ``DATA_KIND`` pointing at an event store / per-user sequence files: the
    keys it names for other data kinds are not handed to the chosen dataset; a table smaller than the store's id
    range is refused with a message."""
    from mlperf_training_b200.data.sequences import write_synthetic_sequences
    from mlperf_training_b200.data.yambda import write_synthetic_event_store
    from mlperf_training_b200.trainer import cli
    root = tmp_path / "data"
    if kind == "yambda":
        write_synthetic_event_store(str(root), 120, 80, 2000, days=3, seed=1)
    else:
        write_synthetic_sequences(str(root), 120, 2000, min_len=20, max_len=60, seed=1)
    monkeypatch.setenv("DATA_KIND", kind)
    monkeypatch.setenv("DATADIR", str(root))
    mode, module, over = _SHIPPED["workloads/hstu/conf/hstu_yambda.yaml"]
    over = [o for o in over if not o.startswith("embedding.rows")] + ["model.max_seq_len=128", "model.num_positions=512"]
    args = [mode, "--config", str(REPO / "workloads/hstu/conf/hstu_yambda.yaml"), "--device", "cpu"]
    assert cli.main(args + [f"modules.{module}.resolved.{o}" for o in over + ["embedding.rows=2000"]]) == 0
    assert "run_stop" in capsys.readouterr().out
    if kind == "yambda":
        with pytest.raises(ValueError, match="too small"):
            cli.main(args + [f"modules.{module}.resolved.{o}" for o in over + ["embedding.rows=500"]])


def test_launcher_reads_shared_settings_and_keeps_caller_values(tmp_path):
    """``run_with_docker.sh`` in host mode for the workload whose system file sources a file of shared settings: the
    shared values (experiment file, trainer mode, seed) arrive, the system file overrides them, the caller overrides
    both, and the trial log is compliant."""
    P = "modules.flux_trainer.resolved"
    over = " ".join(f"{P}.{o}" for o in _SHIPPED["workloads/flux1/conf/flux.1_schnell_t2i-pretrain.yaml"][2])
    env = dict(os.environ, DGXSYSTEM="B200_1x8x32", NGPU="1", NEXP="1", LOGDIR=str(tmp_path), CUDA_VISIBLE_DEVICES="", LR="1e-3",
               PYTHONPATH=str(REPO), EXTRA_OVERRIDES="--device cpu " + over)
    env.pop("SEED", None)
    res = subprocess.run(["bash", str(REPO / "workloads/flux1/run_with_docker.sh")], env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "compliance: SUCCESS" in res.stdout and "RESULT,flux1,," in res.stdout and "seed 10007" in res.stdout
    recs = parse_log(res.stdout)
    lr = [r["value"] for r in recs if r["key"] == "opt_base_learning_rate"]
    gbs = [r["value"] for r in recs if r["key"] == "global_batch_size"]
    assert lr == [1e-3] and gbs == [2]            # the caller's LR beats the file's 2.5e-4; the override beats GBS=256


def test_misspelt_experiment_keys_are_reported():
    import warnings
    from mlperf_training_b200.config.loader import warn_unknown_keys
    from mlperf_training_b200.trainer import flux, hstu
    for path, module, fn in (("workloads/hstu/conf/hstu_yambda.yaml", "hstu_trainer", hstu.run),
                             ("workloads/flux1/conf/flux.1_schnell_t2i-pretrain.yaml", "flux_trainer", flux.run)):
        resolved = loader.load_experiment(REPO / path, env={})["modules"][module]["resolved"]
        with warnings.catch_warnings(record=True) as w:
            warnings.simplefilter("always")
            assert warn_unknown_keys(resolved, fn, "experiment") == [] and not w          # every shipped key is read
            assert warn_unknown_keys(dict(resolved, trian_steps=3), fn, "experiment") == ["trian_steps"]
            assert len(w) == 1 and "trian_steps" in str(w[0].message)


def test_cli_prints_the_resolved_experiment(capsys, monkeypatch):
    import yaml
    from mlperf_training_b200.trainer import cli
    monkeypatch.setenv("GBS", "64")
    rc = cli.main(["pretrain", "--config", str(REPO / "workloads/llama31_8b/conf/llama3.1_8B-pretrain-mxfp8.yaml"), "--print-config",
                   "modules.pre_trainer.resolved.lr=0.5"])
    got = yaml.safe_load(capsys.readouterr().out)
    assert rc == 0 and got["global_batch"] == 64 and got["lr"] == 0.5 and got["model"]["precision"] == "mxfp8"
