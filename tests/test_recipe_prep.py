"""Precision schedule (format mapping, switch step, env override, de-oscillation status) and the
data-preparation tools (packing, metadata, checksums, time-window index)."""
import numpy as np
import pytest
import torch.nn as nn

from mlperf_training_b200.data import prep
from mlperf_training_b200.data.indexed import PackedSFTDataset
from mlperf_training_b200.ops.recipe import PrecisionSchedule, resolve_format


def test_precision_schedule_switch_and_mapping(monkeypatch):
    assert resolve_format("A6W4") == "a6w4" and resolve_format("nvfp4") == "mxfp4" and resolve_format("bf16") == "bf16"
    with pytest.raises(ValueError):
        resolve_format("int3")

    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.precision = "bf16"
            self.sub = nn.Linear(2, 2)
            self.sub.precision = "bf16"
    m = M()
    s = PrecisionSchedule.from_spec({"initial": "bf16", "switch_step": 5, "final": "fp8",
                                     "deosc": {"enabled": True, "start_step": 768}})
    assert s.apply(m, 0) and m.precision == "bf16"
    assert not s.apply(m, 4)
    assert s.apply(m, 5) and m.precision == "fp8" and m.sub.precision == "fp8"
    assert s.log == [(0, "bf16"), (5, "fp8")]
    assert "idle" in s.deosc.status("mxfp8") and s.deosc.status("mxfp4").startswith("deosc: on")
    monkeypatch.setenv("FLUX_FPROP_SWITCH_STEP", "9")
    assert PrecisionSchedule.from_spec({"initial": "a6w4", "switch_step": 5, "final": "bf16"}).phases[1][0] == 9


def test_pack_convert_metadata_hash_verify(tmp_path):
    rng = np.random.default_rng(0)
    samples = [{"input_ids": rng.integers(0, 100, size=n).tolist(), "labels": [-100] * (n // 2) + [1] * (n - n // 2)}
               for n in (30, 9, 17, 12, 5, 33, 20)]
    rows = prep.pack_samples(samples, seq_len=32)
    assert sum(len(r["input_ids"]) for r in rows) == sum(len(s["input_ids"]) for s in samples)
    assert all(len(r["input_ids"]) <= 33 for r in rows) and len(rows) <= 5
    assert all(r["seq_start_id"][0] == 0 and r["seq_start_id"] == sorted(r["seq_start_id"]) for r in rows)
    src = tmp_path / "s.jsonl"
    import json
    src.write_text("\n".join(json.dumps(s) for s in samples))
    n = prep.convert_sft(str(src), str(tmp_path / "train.npy"), 32)
    assert n == len(rows) and prep.write_metadata(str(tmp_path / "train.npy"), str(tmp_path / "meta.jsonl")) == n
    ds = PackedSFTDataset(str(tmp_path / "train.npy"), 32, str(tmp_path / "meta.jsonl"))
    assert len(ds) == n and len(ds.metadata) == n
    manifest = tmp_path / "sums.md5"
    manifest.write_text("\n".join(f"{d}  {name}" for d, name in prep.hash_directory(str(tmp_path)) if name != "sums.md5"))
    assert prep.verify_directory(str(tmp_path), str(manifest)) == []
    (tmp_path / "meta.jsonl").write_text("tampered")
    assert prep.verify_directory(str(tmp_path), str(manifest)) == ["meta.jsonl"]


def test_window_index_is_ordered_and_deterministic():
    ts = np.array([50, 10, 70, 11, 130, 12, 200, 131])
    idx = prep.build_window_index(ts, window_seconds=60, holdout=0.25, salt=7)
    assert ts[idx["order"]].tolist() == sorted(ts.tolist())
    assert idx["window_start"].tolist() == [0, 4, 5, 7] and idx["window_id"].tolist() == [0, 1, 2, 3]
    again = prep.build_window_index(ts, 60, 0.25, 7)
    assert np.array_equal(idx["holdout"], again["holdout"])
    big = prep.build_window_index(np.arange(20000), 100, holdout=0.1, salt=1)
    assert 0.07 < big["holdout"].mean() < 0.13


def test_first_and_last_layers_stay_in_bf16(monkeypatch):
    import torch
    from mlperf_training_b200.models.gpt import GPT, GPTConfig
    from mlperf_training_b200.ops import functional as F
    cfg = GPTConfig(n_layers=4, hidden=32, n_heads=2, n_kv_heads=1, head_dim=16, ffn_hidden=64, vocab_size=64, seq_len=8, dtype="fp32",
                    precision="mxfp8", bf16_first_layers=1, bf16_last_layers=2)
    m = GPT(cfg, seed=0)
    assert [b.force_bf16 for b in m.blocks] == [True, False, True, True]
    assert [b.mlp.force_bf16 for b in m.blocks] == [True, False, True, True]
    seen = []
    real = F.norm_linear

    def spy(*a, **kw):
        seen.append(kw.get("precision"))
        return real(*a, **kw)
    monkeypatch.setattr(F, "norm_linear", spy)
    tok = torch.randint(0, 64, (1, 9))
    m(tok[:, :-1], tok[:, 1:]).backward()
    # per layer: the qkv projection and the gate/up projection
    assert seen == ["bf16", "bf16", "mxfp8", "mxfp8", "bf16", "bf16", "bf16", "bf16"]


def test_activation_offload_gives_the_same_gradients():
    import torch
    from mlperf_training_b200.models.gpt import GPT, GPTConfig
    base = dict(n_layers=3, hidden=32, n_heads=2, n_kv_heads=1, head_dim=16, ffn_hidden=64, vocab_size=64, seq_len=8, dtype="fp32")
    tok = torch.randint(0, 64, (2, 9), generator=torch.Generator().manual_seed(0))
    grads = []
    for mode, layers in (("none", 0), ("offload", 0), ("offload", 2), ("full", 0)):
        m = GPT(GPTConfig(**base, recompute=mode, recompute_layers=layers), seed=2)
        loss = m(tok[:, :-1], tok[:, 1:])
        loss.backward()
        grads.append((float(loss), [p.grad.clone() if p.grad is not None else p.main_grad.clone() for p in m.parameters()]))
    for l, g in grads[1:]:
        assert l == grads[0][0]
        assert all(torch.allclose(a, b, atol=1e-7) for a, b in zip(g, grads[0][1]))
