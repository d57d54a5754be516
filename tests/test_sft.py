"""LoRA SFT runs: packed samples on one CPU process (only adapters move, token-weighted eval, MLLOG
compliance) and a tensor-parallel posttrain run through the CLI on two gloo ranks."""
import io
import os
import subprocess
import sys

import torch

from mlperf_training_b200.data.indexed import write_packed_sft
from mlperf_training_b200.mllog import check_compliance
from mlperf_training_b200.trainer.sft import run

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MODEL = dict(n_layers=2, hidden=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn_hidden=128, vocab_size=256, seq_len=32,
             dtype="fp32", lora_rank=4, lora_alpha=8.0, lora_dropout=0.0)


def test_packed_sft_run_trains_only_adapters(tmp_path):
    g = torch.Generator().manual_seed(0)
    samples = []
    for _ in range(24):
        n = int(torch.randint(20, 34, (1,), generator=g))
        ids = torch.randint(0, 256, (n,), generator=g)
        mask = torch.zeros(n, dtype=torch.int64)
        mask[n // 2:] = 1
        samples.append({"input_ids": ids.numpy(), "loss_mask": mask.numpy(), "seq_start_id": [0]})
    write_packed_sft(str(tmp_path / "train.npy"), samples, str(tmp_path / "meta.jsonl"))
    exp = dict(model=MODEL, global_batch=4, micro_batch=2, train_iters=6, lr=5e-3, eval_interval=2, eval_iters=2,
               skip_evals=1, target_eval_loss=0.0, warmup_train_steps=1, warmup_eval_steps=0,
               data=dict(kind="packed_sft", path=str(tmp_path / "train.npy"), metadata=str(tmp_path / "meta.jsonl")))
    out = run(exp, device="cpu", stream=io.StringIO())
    tr = out["trainer"]
    names = [n for b in tr.engine.buckets for n, _ in b.params]
    assert names and all("lora" in n for n in names)
    assert all(l == l for l in out["losses"]) and out["eval_loss"] is not None
    assert any(float(blk.lora_qkv.b.abs().sum()) > 0 for blk in tr.model.blocks)      # B left its zero init
    assert check_compliance(out["records"]) == []
    evals = [r for r in out["records"] if r["key"] == "eval_accuracy"]
    assert len(evals) == 2                                                            # 3 intervals, first one skipped


def test_posttrain_cli_tensor_parallel_gloo(tmp_path):
    yaml = tmp_path / "exp.yaml"
    yaml.write_text("""
modules:
  post_trainer:
    framework: b200
    overrides:
      global_batch: 2
      micro_batch: 1
      train_iters: 3
      tensor_parallel: 2
      tp_comm_overlap: nccl
      eval_interval: 0
      warmup_train_steps: 0
      model: {n_layers: 2, hidden: 64, n_heads: 4, n_kv_heads: 2, head_dim: 16, ffn_hidden: 128, vocab_size: 256,
              seq_len: 32, dtype: fp32, lora_rank: 4, lora_dropout: 0.0}
      data: {kind: synthetic, loss_last: 8}
""")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29647", "-m", "mlperf_training_b200.trainer.cli",
                        "posttrain", "--config", str(yaml), "--device", "cpu"], env=env, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "run_stop" in r.stdout and "train_loss" in r.stdout


def test_eod_mask_loss_drops_positions_after_document_ends():
    """``eod_mask_loss``: the label is -100 wherever the input token is the end-of-document token; the run loop's loss
    is then the mean over the remaining positions."""
    import io

    import torch

    from mlperf_training_b200.trainer.loop import eod_masked, run
    tok = torch.tensor([[5, 9, 2, 7, 9, 9, 1]])
    x, y = eod_masked(tok, 9)
    assert x.tolist() == [[5, 9, 2, 7, 9, 9]] and y.tolist() == [[9, -100, 7, 9, -100, -100]]
    x2, y2 = eod_masked((tok[:, :-1], torch.tensor([[-100, -100, 7, 9, 9, 1]])), 9)      # explicit labels keep their own mask
    assert y2.tolist() == [[-100, -100, 7, 9, -100, -100]]
    tiny = dict(n_layers=2, hidden=32, n_heads=2, n_kv_heads=1, head_dim=16, ffn_hidden=64, vocab_size=8, seq_len=32, dtype="fp32")
    base = dict(model=tiny, global_batch=2, micro_batch=1, train_iters=2, lr=1e-3, lr_warmup_iters=1)
    a = run(dict(base), device="cpu", stream=io.StringIO())
    b = run(dict(base, eod_mask_loss=1, eod_token=3), device="cpu", stream=io.StringIO())
    assert a["losses"][0] != b["losses"][0] and abs(a["losses"][0] - b["losses"][0]) < 0.2   # an eighth of the positions left out
