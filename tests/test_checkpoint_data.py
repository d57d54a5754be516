"""Checkpoint manager (atomic directories, pruning, cadence, resume position, split contract),
Megatron name mapping and torch_dist round trip, indexed / packed datasets, warm-up restore, a
fault-injected GPT run that resumes, and a FLUX (MMDiT) run on CPU."""
import io

import numpy as np
import pytest
import torch

from mlperf_training_b200.checkpoint import megatron as MG
from mlperf_training_b200.checkpoint.manager import (CheckpointManager, resume_position, select_checkpoint_reason,
                                                      validate_split_contract)
from mlperf_training_b200.data.indexed import (GPTSampleDataset, MMapIndexedDataset, PackedSFTDataset, SyntheticTokens,
                                               write_indexed_dataset, write_packed_sft)
from mlperf_training_b200.mllog import check_compliance
from mlperf_training_b200.models.gpt import GPT, GPTConfig

TINY = dict(n_layers=2, hidden=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn_hidden=128, vocab_size=256, seq_len=32,
            dtype="fp32")


def test_manager_atomic_save_prune_and_load(tmp_path):
    m = CheckpointManager(str(tmp_path / "ck"), keep_last=2)
    assert not m.present() and m.load() is None
    (tmp_path / "ck").mkdir()
    (tmp_path / "ck" / "7.tmp").mkdir()                       # a crashed save
    for step in (10, 20, 30):
        m.save(step, dense={"w": torch.full((3,), float(step))}, optim_shard={"m": torch.ones(2) * step},
               meta={"samples": step * 4, "window": 0, "batch_idx_in_window": step})
    assert m.steps() == [20, 30] and not (tmp_path / "ck" / "7.tmp").exists()
    assert (tmp_path / "ck" / "latest_checkpointed_iteration.txt").read_text() == "30"
    ck = m.load()
    assert ck["meta"]["step"] == 30 and float(ck["dense"]["w"][0]) == 30.0 and float(ck["optim"]["m"][0]) == 30.0
    torch.manual_seed(123)
    m.save(40, dense=None, optim_shard=None, meta={})
    a = torch.rand(3)
    CheckpointManager.restore_rng(m.load(40)["rng"])
    assert torch.equal(torch.rand(3), a)


def test_cadence_resume_position_and_contract():
    kw = dict(batch_in_window=0, elapsed_since_last_s=0.0)
    assert select_checkpoint_reason(global_step=100, every_steps=50, **kw) == "global_step"
    assert select_checkpoint_reason(global_step=101, every_steps=50, **kw) is None
    assert select_checkpoint_reason(global_step=3, batch_in_window=8, elapsed_since_last_s=0, every_window_batches=4) == "in_window"
    assert select_checkpoint_reason(global_step=3, batch_in_window=1, elapsed_since_last_s=99, every_seconds=60) == "wall_clock"
    assert select_checkpoint_reason(global_step=3, window_end=True, **kw) == "window"
    assert resume_position(None, 8)["cold_start"]
    assert resume_position({"window": 2, "batch_idx_in_window": 5}, 8) == {"window": 2, "skip_batches": 5, "skip_samples": 40,
                                                                           "cold_start": False}
    assert resume_position({"window": 2, "batch_idx_in_window": -1}, 8)["window"] == 3
    validate_split_contract({"salt": 1, "world": 8}, {"salt": 1, "world": 8})
    with pytest.raises(RuntimeError):
        validate_split_contract({"salt": 1, "world": 8}, {"salt": 2, "world": 8})
    validate_split_contract({"salt": 1}, {"salt": 2}, allow_mismatch=True)


def test_megatron_names_qkv_layout_and_torch_dist_roundtrip(tmp_path):
    cfg = GPTConfig(**TINY)
    a = GPT(cfg, seed=1)
    state = MG.to_megatron_state(a)
    assert "decoder.layers.0.self_attention.linear_qkv.weight" in state
    assert "embedding.word_embeddings.weight" in state and "output_layer.weight" in state
    for name in state:
        assert MG.megatron_name(MG.local_name(name)) == name
    w = a.blocks[0].w_qkv.detach()
    meg = MG.qkv_to_megatron(w, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim)
    assert meg.shape == w.shape and not torch.equal(meg, w)
    assert torch.equal(MG.qkv_from_megatron(meg, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim), w)
    # first query group of Megatron's layout: q heads of group 0, then its k head, then its v head
    hd, g = cfg.head_dim, cfg.n_heads // cfg.n_kv_heads
    assert torch.equal(meg[: g * hd], w[: g * hd])
    assert torch.equal(meg[g * hd:(g + 1) * hd], w[cfg.n_heads * hd: cfg.n_heads * hd + hd])
    root = MG.save_torch_dist(a, str(tmp_path / "base"), iteration=0)
    assert (root / ".metadata").exists() and (tmp_path / "base" / "latest_checkpointed_iteration.txt").exists()
    b = GPT(cfg, seed=2)
    MG.load_torch_dist(b, str(tmp_path / "base"))
    for (n, p), (_, q) in zip(a.named_parameters(), b.named_parameters()):
        assert torch.equal(p, q), n


def test_indexed_dataset_and_gpt_samples(tmp_path):
    rng = np.random.default_rng(0)
    docs = [rng.integers(0, 1000, size=int(n), dtype=np.int32) for n in rng.integers(5, 60, size=40)]
    prefix = str(tmp_path / "c4")
    write_indexed_dataset(prefix, docs)
    ds = MMapIndexedDataset(prefix)
    assert len(ds) == 40 and ds.num_tokens == sum(len(d) for d in docs)
    assert np.array_equal(ds[7], docs[7])
    flat = np.concatenate(docs)
    assert np.array_equal(ds.tokens(33, 50), flat[33:83])
    g = GPTSampleDataset([prefix], None, seq_len=16, seed=3)
    b0 = g.batch(0, 0, 2, 3)
    assert b0.shape == (3, 17) and b0.dtype == torch.int64
    assert torch.equal(b0, GPTSampleDataset([prefix], None, seq_len=16, seed=3).batch(0, 0, 2, 3))     # deterministic
    assert not torch.equal(b0, g.batch(0, 1, 2, 3))                                                    # rank slices differ


def test_packed_sft_and_synthetic_labels(tmp_path):
    samples = [{"input_ids": np.arange(10), "loss_mask": np.array([0] * 6 + [1] * 4), "seq_start_id": [0, 6]},
               {"input_ids": np.arange(40), "loss_mask": np.ones(40, dtype=np.int64), "seq_start_id": [0]}]
    write_packed_sft(str(tmp_path / "t.npy"), samples, str(tmp_path / "m.jsonl"))
    ds = PackedSFTDataset(str(tmp_path / "t.npy"), seq_len=16, metadata_path=str(tmp_path / "m.jsonl"))
    tok, lab, starts = ds[0]
    assert tok.shape == (16,) and lab.shape == (16,)
    assert lab[:5].eq(-100).all() and lab[5:9].tolist() == [6, 7, 8, 9] and lab[9:].eq(-100).all()   # short sample is padded
    tok, lab, _ = ds[1]
    assert lab.tolist() == list(range(1, 17))                                                         # long sample is cut
    t, l = ds.batch(0, 0, 1, 2)
    assert t.shape == (2, 16) and l.shape == (2, 16)
    syn = SyntheticTokens(100, 16, seed=1, loss_last=4)
    b = syn.batch(3, 0, 1, 2)
    lab = syn.labels(b)
    assert lab[:, :12].eq(-100).all() and torch.equal(lab[:, 12:], b[:, 13:])


def test_warmup_restores_everything():
    from mlperf_training_b200.parallel.engine import OptimConfig
    from mlperf_training_b200.trainer.pretrain import PretrainTrainer, TrainConfig
    from mlperf_training_b200.trainer.warmup import run_synthetic_warmup
    tr = PretrainTrainer(GPTConfig(**TINY), OptimConfig(lr=1e-2), TrainConfig(micro_batch=1, local_batch=2), "cpu")
    before = [b.param_buf.clone() for b in tr.engine.buckets]
    run_synthetic_warmup(tr, train_steps=2, eval_steps=1)
    assert tr.step_idx == 0 and tr.engine.step_count == 0
    for b, p0 in zip(tr.engine.buckets, before):
        assert torch.equal(b.param_buf, p0)
        assert float(b.m.abs().sum()) == 0 and float(b.v.abs().sum()) == 0 and float(b.grad_buf.abs().sum()) == 0


def test_gpt_run_die_at_step_then_resume_matches_uninterrupted(tmp_path):
    from mlperf_training_b200.trainer.loop import run
    base = dict(model=TINY, global_batch=2, micro_batch=1, train_iters=6, lr=3e-3, lr_warmup_iters=2, warmup_train_steps=0)
    ref = run(dict(base), device="cpu", stream=io.StringIO())
    exp = dict(base, checkpoint_dir=str(tmp_path / "ck"), die_at_step=3, mllog_file=str(tmp_path / "ml.log"))
    with pytest.raises(SystemExit) as ex:
        run(dict(exp), device="cpu", stream=io.StringIO())
    assert ex.value.code == 42
    exp["die_at_step"] = 0
    out = run(dict(exp), device="cpu", stream=io.StringIO())
    assert out["steps"] == 3
    assert abs(out["losses"][-1] - ref["losses"][-1]) < 1e-5
    lines = (tmp_path / "ml.log").read_text().splitlines()
    assert sum("run_start" in l for l in lines) == 1 and sum("run_stop" in l for l in lines) == 1


def test_flux_run_learns_on_cpu():
    from mlperf_training_b200.trainer.flux import run
    out = run(dict(model=dict(preset="tiny-mmdit"), global_batch=4, train_iters=12, lr=2e-3, eval_every_samples=24,
                   prompt_dropout=0.0), device="cpu", stream=io.StringIO())
    assert all(l == l for l in out["losses"]) and out["eval_loss"] is not None
    assert check_compliance(out["records"]) == []
    # flow matching on a fixed batch: the velocity target has a learnable part (-x0), the loss must fall
    from mlperf_training_b200.models.mmdit import tiny_mmdit
    from mlperf_training_b200.parallel.engine import OptimConfig
    from mlperf_training_b200.trainer.flux import FluxTrainer, SyntheticFluxData
    cfg = tiny_mmdit()
    tr = FluxTrainer(cfg, OptimConfig(lr=3e-3, weight_decay=0.0), "cpu", 4, prompt_dropout=0.0)
    b = SyntheticFluxData(cfg).batch(0, 0, 4)
    ls = [tr.train_step(b) for _ in range(40)]
    assert sum(ls[-5:]) < 0.9 * sum(ls[:5])


def test_async_checkpoint_and_gauc(tmp_path):
    from mlperf_training_b200.utils.metrics import exact_auc, grouped_auc
    m = CheckpointManager(str(tmp_path / "ck"), keep_last=2)
    w = torch.arange(6.0)
    assert m.save_async(5, dense={"w": w}, optim_shard={"m": torch.ones(2)}, meta={"samples": 20}) is None
    w.add_(100)                                            # the snapshot was taken before this change
    assert m.finalize_async() == m.path(5) and m.finalize_async() is None
    ck = m.load()
    assert ck["meta"]["step"] == 5 and torch.equal(ck["dense"]["w"], torch.arange(6.0))
    m.save_async(6, dense={"w": w}, optim_shard=None, meta={})
    m.save_async(7, dense={"w": w}, optim_shard=None, meta={})        # finalises 6 first
    m.finalize_async()
    assert m.steps() == [6, 7]
    s = torch.tensor([0.9, 0.1, 0.8, 0.2, 0.3, 0.7])
    y = torch.tensor([1.0, 0.0, 0.0, 1.0, 1.0, 1.0])
    g = torch.tensor([0, 0, 1, 1, 2, 2])
    assert grouped_auc(s, y, g) == (2 * exact_auc(s[:2], y[:2]) + 2 * exact_auc(s[2:4], y[2:4])) / 4    # group 2 has one class


def test_run_loop_monitors(tmp_path):
    """Async checkpoints, replica check, straggler detector and the performance log inside a run."""
    import json
    from mlperf_training_b200.trainer.loop import run
    out = run(dict(model=TINY, global_batch=2, micro_batch=1, train_iters=4, warmup_train_steps=0, checkpoint_dir=str(tmp_path / "ck"),
                   checkpoint_every=2, async_checkpoint=True, check_replicas_every=2, straggler_interval=2,
                   perf_jsonl=str(tmp_path / "perf.jsonl")), device="cpu", stream=io.StringIO())
    assert out["steps"] == 4
    assert CheckpointManager(str(tmp_path / "ck")).steps() == [2, 4]
    lines = [json.loads(l) for l in (tmp_path / "perf.jsonl").read_text().splitlines()]
    assert len(lines) == 4 and lines[-1]["step"] == 4 and lines[-1]["samples_per_s"] > 0


def test_flux_run_warmup_leaves_no_trace_and_resume_matches(tmp_path):
    from mlperf_training_b200.trainer.flux import run
    base = dict(model=dict(preset="tiny-mmdit"), global_batch=2, train_iters=5, lr=2e-3, lr_warmup_iters=2, eval_every_samples=6)
    ref = run(dict(base), device="cpu", stream=io.StringIO())
    warm = run(dict(base, warmup_train_steps=2, warmup_eval_steps=1), device="cpu", stream=io.StringIO())
    assert warm["losses"] == ref["losses"] and warm["eval_loss"] == ref["eval_loss"]
    exp = dict(base, checkpoint_dir=str(tmp_path / "ck"), checkpoint_every=2, keep_last=1, die_at_step=3,
               mllog_file=str(tmp_path / "ml.log"))
    with pytest.raises(SystemExit) as ex:
        run(dict(exp), device="cpu", stream=io.StringIO())
    assert ex.value.code == 42
    assert CheckpointManager(str(tmp_path / "ck")).steps() == [3]                      # keep_last = 1 dropped step 2
    out = run(dict(exp, die_at_step=0), device="cpu", stream=io.StringIO())
    assert out["steps"] == 2 and out["losses"] == ref["losses"][3:]
    lines = (tmp_path / "ml.log").read_text().splitlines()
    assert sum("run_start" in l for l in lines) == 1 and sum("run_stop" in l for l in lines) == 1


def test_mmdit_recompute_gives_the_same_gradients():
    from mlperf_training_b200.models.mmdit import MMDiT, tiny_mmdit
    cfg = tiny_mmdit()
    plain = MMDiT(cfg, device="cpu", seed=4)
    import dataclasses
    rec = MMDiT(dataclasses.replace(cfg, recompute="full", recompute_ratio=0.5), device="cpu", seed=4)
    rec.load_state_dict(plain.state_dict())
    g = torch.Generator().manual_seed(0)
    lat = torch.randn(2, cfg.img_tokens, cfg.in_channels, generator=g)
    txt = torch.randn(2, cfg.txt_tokens, cfg.txt_dim, generator=g)
    vec = torch.randn(2, cfg.vec_dim, generator=g)
    for m in (plain, rec):
        m.loss(lat, txt, vec, generator=torch.Generator().manual_seed(1)).backward()
    for (n, p), (_, q) in zip(plain.named_parameters(), rec.named_parameters()):
        gp = p.grad if p.grad is not None else getattr(p, "main_grad", None)
        gq = q.grad if q.grad is not None else getattr(q, "main_grad", None)
        assert (gp is None) == (gq is None), n
        if gp is not None:
            assert torch.allclose(gp, gq, atol=1e-6), n


def test_flux_run_on_pre_encoded_dataset(tmp_path):
    import numpy as np
    from mlperf_training_b200.data.flux_encoded import EncodedFluxData, write_encoded_dataset
    from mlperf_training_b200.models.mmdit import patchify, tiny_mmdit, unpatchify
    from mlperf_training_b200.trainer.flux import run
    cfg = tiny_mmdit()
    side = int(round((cfg.img_tokens) ** 0.5)) * 2
    C = cfg.in_channels // 4
    rng = np.random.default_rng(0)
    n = 12
    lat = rng.standard_normal((n, C, side, side)).astype(np.float16)
    write_encoded_dataset(str(tmp_path / "enc"), lat, rng.standard_normal((n, cfg.txt_tokens, cfg.txt_dim)).astype(np.float16),
                          rng.standard_normal((n, cfg.vec_dim)).astype(np.float16),
                          empty_t5=np.zeros((cfg.txt_tokens, cfg.txt_dim), np.float16) + 0.5, empty_clip=np.zeros(cfg.vec_dim, np.float16) - 0.5)
    ds = EncodedFluxData(str(tmp_path / "enc"), cfg, seed=1)
    a, b = ds.indices(0, 0, 2, world=2), ds.indices(0, 1, 2, world=2)
    assert not set(a) & set(b) and ds.steps_per_epoch(2, 2) == 3
    seen = np.concatenate([ds.indices(s, r, 2, 2) for s in range(3) for r in range(2)])
    assert sorted(seen.tolist()) == list(range(n))                                  # an epoch visits every sample once
    assert ds.indices(3, 0, 2, 2).tolist() != a.tolist() or ds.indices(4, 0, 2, 2).tolist() != ds.indices(1, 0, 2, 2).tolist()
    x, t5, clip = ds.batch(0, 0, 2)
    assert x.shape == (2, cfg.img_tokens, cfg.in_channels) and t5.shape == (2, cfg.txt_tokens, cfg.txt_dim)
    back = unpatchify(patchify(torch.from_numpy(lat[:2].astype(np.float32))), C, side // 2)
    assert torch.equal(back, torch.from_numpy(lat[:2].astype(np.float32)))
    with pytest.raises(ValueError):
        EncodedFluxData(str(tmp_path / "enc"), __import__("dataclasses").replace(cfg, txt_tokens=cfg.txt_tokens * 2))
    out = run(dict(model=dict(preset="tiny-mmdit"), global_batch=2, train_iters=4, lr=2e-3, eval_every_samples=4, prompt_dropout=0.5,
                   data=dict(kind="encoded", path=str(tmp_path / "enc"))), device="cpu", stream=io.StringIO())
    assert len(out["losses"]) == 4 and all(l == l for l in out["losses"]) and out["eval_loss"] is not None
    assert out["trainer"].empty_txt is not None and float(out["trainer"].empty_txt.mean()) == 0.5


def test_torch_dist_checkpoint_loads_into_pipeline_stages(tmp_path):
    import torch.nn as nn
    from mlperf_training_b200.parallel.pipeline import GPTStage
    cfg = GPTConfig(**{**TINY, "n_layers": 5})
    full = GPT(cfg, seed=1)
    MG.save_torch_dist(full, str(tmp_path / "base"), iteration=0)
    # two plain stages (3 + 2 layers) ...
    for s in range(2):
        stage = GPTStage(cfg, s, 2)
        info = MG.load_torch_dist(stage, str(tmp_path / "base"))
        assert info["missing"] == []
        for blk, i in zip(stage.blocks, stage.layers):
            for (n, p), (_, q) in zip(blk.named_parameters(), full.blocks[i].named_parameters()):
                assert torch.equal(p, q), (s, i, n)
        if stage.first:
            assert torch.equal(stage.embed, full.embed)
        if stage.last:
            assert torch.equal(stage.lm_head, full.lm_head) and torch.equal(stage.final_norm, full.final_norm)
    # ... and the two chunks a rank owns under interleaved stages (virtual stages 1 and 3 of 4)
    chunks = nn.ModuleList([GPTStage(cfg, 1, 4), GPTStage(cfg, 3, 4)])
    MG.load_torch_dist(chunks, str(tmp_path / "base"))
    for ch in chunks:
        for blk, i in zip(ch.blocks, ch.layers):
            assert torch.equal(blk.w_qkv, full.blocks[i].w_qkv)
    assert torch.equal(chunks[1].lm_head, full.lm_head)
    names = [n for n, _ in MG.global_named_parameters(chunks)]
    assert len(names) == len(set(names)) and all(n in dict(full.named_parameters()) for n in names)


def test_hf_llama_directory_converts_to_a_loadable_torch_dist_checkpoint(tmp_path):
    """Hugging Face names / split projections -> fused GPT parameters -> torch_dist files that load back."""
    import json

    import torch

    from mlperf_training_b200.checkpoint.megatron import load_torch_dist
    from mlperf_training_b200.data.prep import convert_hf_llama
    from mlperf_training_b200.models.gpt import GPT, PRESETS
    cfg = PRESETS["llama2-70b"]()
    small = dict(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, intermediate_size=128, vocab_size=96)
    hd = cfg.head_dim = 16
    g = torch.Generator().manual_seed(0)
    hf = {"model.embed_tokens.weight": torch.randn(96, 64, generator=g), "model.norm.weight": torch.ones(64),
          "lm_head.weight": torch.randn(96, 64, generator=g)}
    for i in range(2):
        p = f"model.layers.{i}."
        hf[p + "input_layernorm.weight"] = torch.ones(64)
        hf[p + "post_attention_layernorm.weight"] = torch.ones(64)
        hf[p + "self_attn.q_proj.weight"] = torch.randn(4 * hd, 64, generator=g)
        hf[p + "self_attn.k_proj.weight"] = torch.randn(2 * hd, 64, generator=g)
        hf[p + "self_attn.v_proj.weight"] = torch.randn(2 * hd, 64, generator=g)
        hf[p + "self_attn.o_proj.weight"] = torch.randn(64, 4 * hd, generator=g)
        hf[p + "mlp.gate_proj.weight"] = torch.randn(128, 64, generator=g)
        hf[p + "mlp.up_proj.weight"] = torch.randn(128, 64, generator=g)
        hf[p + "mlp.down_proj.weight"] = torch.randn(64, 128, generator=g)
    src = tmp_path / "hf"
    src.mkdir()
    (src / "config.json").write_text(json.dumps(small))
    torch.save(hf, src / "pytorch_model.bin")
    import mlperf_training_b200.models.gpt as G
    orig = G.PRESETS["llama2-70b"]
    G.PRESETS["llama2-70b"] = lambda: G.GPTConfig(head_dim=16, dtype="fp32", seq_len=32)
    try:
        out = convert_hf_llama(str(src), str(tmp_path / "ckpt"), dtype="fp32")
        c = G.PRESETS["llama2-70b"]()
        for k, v in dict(n_layers=2, hidden=64, n_heads=4, n_kv_heads=2, ffn_hidden=128, vocab_size=96).items():
            setattr(c, k, v)
        m = GPT(c, device="cpu", seed=5)
        load_torch_dist(m, str(tmp_path / "ckpt"))
    finally:
        G.PRESETS["llama2-70b"] = orig
    assert "iter_0000000" in out
    assert torch.equal(m.blocks[1].w_qkv[:4 * hd], hf["model.layers.1.self_attn.q_proj.weight"])
    assert torch.equal(m.blocks[0].mlp.w_gate_up[128:], hf["model.layers.0.mlp.up_proj.weight"])
    assert torch.equal(m.lm_head, hf["lm_head.weight"])
