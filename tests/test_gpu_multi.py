"""Multi-GPU tests (need >= 2 GPUs on the box): each case runs a worker script under torchrun."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = Path(__file__).resolve().parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(worker: str, nproc: int = 2, timeout: int = 600, extra_env: dict | None = None, args=()):
    # B200_TEST_NPROC=8 runs the same workers on every GPU of the box (the W = 8 result checks)
    nproc = min(int(os.environ.get("B200_TEST_NPROC", nproc)), torch.cuda.device_count())
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), str(HERE / "multi" / worker), *args]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_zero_step_matches_nccl():
    res = _run("zero_fused_worker.py")
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "RESULT ok=True" in res.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("comm", ["nccl", "fused"])
def test_sharded_embedding_two_gpus(comm):
    res = _run("embedding_worker.py", args=("nccl", comm))
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("comm,lora", [("nccl", False), ("fused", False), ("fused", True)])
def test_tensor_parallel_gpt_two_gpus(comm, lora):
    res = _run("tp_worker.py", args=("nccl", comm) + (("lora",) if lora else ()))
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "RESULT rank 0 ok=True" in res.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tensor_parallel_lora_frozen_base_fp8():
    """LoRA over a frozen base whose tensor-parallel linears run the fused kernels on per-tensor FP8 operands."""
    res = _run("tp_worker.py", args=("nccl", "fused", "lora", "fp8"))
    assert res.returncode == 0 and res.stdout.count("ok=True") >= 2, res.stdout[-3000:] + res.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("precision", ["bf16", "mxfp8"])
def test_fused_expert_dispatch_matches_all_to_all(precision):
    res = _run("moe_fused_worker.py", args=(precision,))
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "RESULT rank 0 ok=True" in res.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_context_parallel_attention_two_gpus():
    res = _run("cp_worker.py", args=("nccl",))
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "RESULT rank 0 ok=True" in res.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_pipeline_parallel_two_gpus():
    res = _run("pp_worker.py", args=("nccl",))
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "RESULT rank 0 ok=True" in res.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_moe_model_expert_parallel_fused_vs_nccl():
    res = _run("moe_ep_worker.py")
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "RESULT rank 0 ok=True" in res.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("comm,precision", [("nccl", "bf16"), ("fused", "mxfp8")])
def test_sharded_parameter_engine_matches_replicated_engine(comm, precision):
    """ZeRO-3 over NCCL collectives and over the NVLS kernels (multimem.st gather, multimem.ld_reduce
    reduce-scatter) against the replicated-parameter engine."""
    res = _run("zero3_worker.py", args=("nccl", comm, precision), extra_env={"NCCL_NVLS_ENABLE": "1"} if comm == "fused" else None)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "RESULT rank 0 ok=True" in res.stdout
