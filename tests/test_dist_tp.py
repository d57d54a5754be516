"""Tensor + sequence parallel GPT on gloo (world 2): loss and gradient-norm parity with the
unsharded model, with and without LoRA; mesh arithmetic."""
import os
import subprocess
import sys

import pytest

from mlperf_training_b200.parallel.mesh import MeshSpec, coords, group_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("extra", [(), ("nccl", "lora")])
def test_tp_parity_gloo(extra):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29643",
                        os.path.join(ROOT, "tests", "multi", "tp_worker.py"), "gloo", *extra],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RESULT rank 0 ok=True" in r.stdout


def test_mesh_groups_partition_the_world():
    spec = MeshSpec(tp=2, pp=2, ep=2)
    g = group_ranks(spec, 16)
    for dim, lists in g.items():
        flat = sorted(r for l in lists for r in l)
        assert flat == list(range(16)), dim
    assert g["tp"][0] == [0, 1] and g["pp"][0] == [0, 8]
    assert all(len(l) == 2 for l in g["ep"]) and all(len(l) == 4 for l in g["dp"])
    assert coords(13, spec, 16) == {"tp": 1, "cp": 0, "dp": 2, "pp": 1}
    with pytest.raises(ValueError):
        group_ranks(MeshSpec(tp=3), 16)


@pytest.mark.parametrize("stages", [2, 3])
def test_pipeline_1f1b_parity_gloo(stages):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={stages}",
                        "--master-addr", "127.0.0.1", "--master-port", "29653",
                        os.path.join(ROOT, "tests", "multi", "pp_worker.py"), "gloo"],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RESULT rank 0 ok=True" in r.stdout


@pytest.mark.parametrize("ranks,chunks,micro", [(2, 2, 4), (3, 2, 6), (2, 3, 2)])
def test_interleaved_pipeline_parity_gloo(ranks, chunks, micro):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}",
                        "--master-addr", "127.0.0.1", "--master-port", "29663",
                        os.path.join(ROOT, "tests", "multi", "vpp_worker.py"), str(chunks), str(micro)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RESULT rank 0 ok=True" in r.stdout


def test_stage_layer_split():
    from mlperf_training_b200.parallel.pipeline import stage_layers
    assert [list(stage_layers(10, 4, s)) for s in range(4)] == [[0, 1, 2], [3, 4, 5], [6, 7], [8, 9]]
    assert sum(len(stage_layers(80, 8, s)) for s in range(8)) == 80


@pytest.mark.parametrize("world", [3, 2])          # world 2 divides the 2 kv heads: the Ulysses exchange runs too
def test_context_parallel_attention_gloo(world):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", "29658",
                        os.path.join(ROOT, "tests", "multi", "cp_worker.py"), "gloo", "ring"],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RESULT rank 0 ok=True" in r.stdout


def test_tensor_x_context_parallel_matches_plain_trainer_gloo():
    """Tensor 2 x context 2 on four ranks (all-gather and ring forms, masked labels) against the plain trainer."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
                        "--master-addr", "127.0.0.1", "--master-port", "29677",
                        os.path.join(ROOT, "tests", "multi", "tp_cp_worker.py")],
                       env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("ok=True") == 4


def test_tensor_x_expert_parallel_follows_the_unsplit_model_gloo():
    """Tensor 2 x data 2 with the experts spread over the data-parallel ranks: loss and gradient norm of the unsplit
    mixture-of-experts model, then the run loop on the same mesh."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
                        "--master-addr", "127.0.0.1", "--master-port", "29680",
                        os.path.join(ROOT, "tests", "multi", "tp_ep_worker.py")],
                       env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("ok=True") == 4


def test_tensor_parallel_stages_checkpoint_round_trips_gloo(tmp_path):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
                        "--master-addr", "127.0.0.1", "--master-port", "29681",
                        os.path.join(ROOT, "tests", "multi", "tp_pp_ckpt_worker.py"), str(tmp_path)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("ok=True") == 4


@pytest.mark.parametrize("virtual", [1, 2])
def test_pipeline_x_context_parallel_follows_the_unsplit_model_gloo(virtual):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
                        "--master-addr", "127.0.0.1", "--master-port", "29682",
                        os.path.join(ROOT, "tests", "multi", "pp_cp_worker.py"), str(virtual)],
                       env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("ok=True") == 4


def test_context_x_expert_parallel_follows_the_unsplit_model_gloo():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
                        "--master-addr", "127.0.0.1", "--master-port", "29683",
                        os.path.join(ROOT, "tests", "multi", "cp_ep_worker.py")],
                       env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("ok=True") == 4


def test_bf16_gradient_wire_follows_the_fp32_wire_gloo():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29676",
                        os.path.join(ROOT, "tests", "multi", "bf16_reduce_worker.py")],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("ok=True") == 2


def test_hybrid_sharding_matches_plain_data_parallel_gloo():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
                        "--master-addr", "127.0.0.1", "--master-port", "29659",
                        os.path.join(ROOT, "tests", "multi", "hsdp_worker.py")],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("ok=True") == 4


@pytest.mark.parametrize("virtual", [1, 2])
def test_tensor_parallel_pipeline_stages_follow_the_unsplit_model_gloo(virtual):
    """Tensor 2 x pipeline 2 on four ranks: loss, gradient norm and weights against the unsplit model, then the run loop."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
                        "--master-addr", "127.0.0.1", "--master-port", "29673",
                        os.path.join(ROOT, "tests", "multi", "tp_pp_worker.py"), str(virtual)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("ok=True") == 4


def test_expert_parallel_pipeline_stages_follow_the_unsplit_model_gloo(tmp_path):
    """Pipeline 2 x data 2 with the experts of every stage spread over its replicas: parity with the unsplit
    mixture-of-experts model, then the run loop (straight, exit after a checkpoint, resume)."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
                        "--master-addr", "127.0.0.1", "--master-port", "29675",
                        os.path.join(ROOT, "tests", "multi", "pp_ep_worker.py"), str(tmp_path)],
                       env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("ok=True") == 4


def test_run_loop_over_tensor_x_pipeline_mesh_resumes_gloo(tmp_path):
    """A run that stops after a checkpoint and resumes ends on the losses of the straight run (every rank owns its own
    slices of its own stage: they travel with the rank's optimizer shard)."""
    import json
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    for phase, want_rc in (("straight", 0), ("die", 42), ("resume", 0)):
        r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
                            "--master-addr", "127.0.0.1", "--master-port", "29674",
                            os.path.join(ROOT, "tests", "multi", "pp_loop_worker.py"), str(tmp_path), "2", "1", phase, "2"],
                           env=env, capture_output=True, text=True, timeout=600)
        assert (r.returncode == 0) == (want_rc == 0), r.stdout[-2000:] + r.stderr[-3000:]
    straight = [json.loads((tmp_path / f"straight_rank{r}.json").read_text()) for r in range(4)]
    resumed = [json.loads((tmp_path / f"resume_rank{r}.json").read_text()) for r in range(4)]
    assert all(s["losses"] == straight[0]["losses"] for s in straight)        # one pipeline, one batch: one loss
    for r in range(4):
        assert max(abs(a - b) for a, b in zip(resumed[r]["losses"], straight[r]["losses"][3:])) < 1e-5


@pytest.mark.parametrize("pp,virtual", [(2, 1), (2, 2)])
def test_run_loop_over_pipeline_mesh_resumes_gloo(tmp_path, pp, virtual):
    import json
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)

    def launch(phase, want_rc):
        r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
                            "--master-addr", "127.0.0.1", "--master-port", "29667",
                            os.path.join(ROOT, "tests", "multi", "pp_loop_worker.py"), str(tmp_path), str(pp), str(virtual), phase],
                           env=env, capture_output=True, text=True, timeout=600)
        assert (r.returncode == 0) == (want_rc == 0), r.stdout[-2000:] + r.stderr[-3000:]

    launch("straight", 0)
    launch("die", 42)
    launch("resume", 0)
    straight = [json.loads((tmp_path / f"straight_rank{r}.json").read_text()) for r in range(4)]
    resumed = [json.loads((tmp_path / f"resume_rank{r}.json").read_text()) for r in range(4)]
    assert straight[0]["steps"] == 6 and resumed[0]["steps"] == 3
    for r in range(2):                                      # ranks r and r + 2 are the two stages of one pipeline
        assert straight[r]["losses"] == straight[r + 2]["losses"]
    assert straight[0]["losses"] != straight[1]["losses"]   # the data-parallel replicas see different data
    for r in range(4):
        assert max(abs(a - b) for a, b in zip(resumed[r]["losses"], straight[r]["losses"][3:])) < 1e-5


def test_context_parallel_training_matches_plain_trainer_gloo():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29669",
                        os.path.join(ROOT, "tests", "multi", "cp_train_worker.py")],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "RESULT rank 0 ok=True" in r.stdout and "RESULT rank 1 ok=True" in r.stdout


@pytest.mark.parametrize("writers,readers", [(4, 2), (2, 4)])
def test_resume_on_another_number_of_ranks_recuts_optimizer_state_gloo(tmp_path, writers, readers):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    for n, phase in ((writers, "write"), (readers, "read")):
        r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                            "--master-addr", "127.0.0.1", "--master-port", "29671",
                            os.path.join(ROOT, "tests", "multi", "reshard_worker.py"), str(tmp_path), phase],
                           env=env, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
        assert "RESULT rank 0 ok=True" in r.stdout


@pytest.mark.parametrize("ranks", [2, 4])        # 2: sequence parallel vs plain; 4: hybrid sharding vs plain data parallel
def test_flux_sequence_parallel_and_hybrid_sharding_match_plain_trainer_gloo(ranks):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}",
                        "--master-addr", "127.0.0.1", "--master-port", "29673",
                        os.path.join(ROOT, "tests", "multi", "flux_sp_worker.py")],
                       env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "RESULT rank 0 ok=True" in r.stdout and "RESULT rank 1 ok=True" in r.stdout


def test_run_loop_with_expert_parallel_resumes_gloo(tmp_path):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29675",
                        os.path.join(ROOT, "tests", "multi", "ep_loop_worker.py"), str(tmp_path)],
                       env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "RESULT rank 0 ok=True" in r.stdout and "RESULT rank 1 ok=True" in r.stdout


def test_tensor_parallel_checkpoints_round_trip_and_runs_resume_gloo(tmp_path):
    """Megatron torch_dist files written under tensor parallelism describe full tensors (every rank its slices); a resumed
    tensor-parallel run restores every rank's own slices; a resumed LoRA run reloads its frozen base."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29717",
                        os.path.join(ROOT, "tests", "multi", "tp_resume_worker.py"), str(tmp_path)],
                       env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "RESULT rank 0 ok=True" in r.stdout and "RESULT rank 1 ok=True" in r.stdout


def test_sharded_parameter_engine_matches_replicated_engine_gloo():
    """ZeRO-3: block matrices live as shards, are gathered per block into rotating windows and their
    gradients are reduced per block; losses and parameters follow the replicated-parameter engine."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29733",
                        os.path.join(ROOT, "tests", "multi", "zero3_worker.py"), "gloo"],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "RESULT rank 0 ok=True" in r.stdout and "RESULT rank 1 ok=True" in r.stdout


def test_tensor_parallel_torch_dist_checkpoint_records_shards_gloo(tmp_path):
    """Every tensor-parallel rank writes its own slices with their offsets; the checkpoint loads into the same
    sharding and into an unsharded model."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29649",
                        os.path.join(ROOT, "tests", "multi", "tp_ckpt_worker.py"), str(tmp_path / "ckpt")],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("ok=True") == 2


def test_expert_parallel_torch_dist_checkpoint_records_shards_gloo(tmp_path):
    """Every expert-parallel rank writes its own experts as a block of the stacked expert dimension; the checkpoint
    loads into the same sharding and into a model that holds every expert."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29651",
                        os.path.join(ROOT, "tests", "multi", "ep_ckpt_worker.py"), str(tmp_path / "ckpt")],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("ok=True") == 2
