"""One small GPT training step on the GPU kernels against the same model on the CPU eager path."""
import pytest
import torch

from mlperf_training_b200.models.gpt import GPT, GPTConfig
from mlperf_training_b200.ops import _lib
from mlperf_training_b200.parallel.engine import OptimConfig
from mlperf_training_b200.trainer.pretrain import PretrainTrainer, TrainConfig, synthetic_tokens

pytestmark = pytest.mark.gpu


def _cfg(**kw):
    base = dict(n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn_hidden=512, vocab_size=1024,
                seq_len=256, rope_theta=10000.0)
    base.update(kw)
    return GPTConfig(**base)


@pytest.mark.parametrize("kw", [dict(), dict(head_dim=128, hidden=512), dict(window=128, window_layers="even", sink=True),
                                dict(head_dim=128, hidden=512, precision="mxfp8"),
                                dict(head_dim=128, hidden=512, precision="mxfp8", swiglu_store="fp8")])
def test_loss_and_grads_match_cpu(kw):
    cfg = _cfg(**kw)
    ref = GPT(GPTConfig(**{**cfg.to_dict(), "dtype": "fp32"}), "cpu", seed=1)
    dev = GPT(cfg, "cuda", seed=1)
    with torch.no_grad():
        for (n, p), (_, q) in zip(ref.named_parameters(), dev.named_parameters()):
            q.copy_(p.to(q.dtype))
            p.copy_(q.float().cpu())  # identical (bf16-representable) weights on both sides
    toks = synthetic_tokens(1, 2, cfg.seq_len, cfg.vocab_size, seed=5, pin=False)[0]
    l_ref = ref(toks[:, :-1], toks[:, 1:])
    l_ref.backward()
    d_toks = toks.cuda()
    l_dev = dev(d_toks[:, :-1], d_toks[:, 1:])
    l_dev.backward()
    torch.cuda.synchronize()
    _lib.check_status("train step")
    assert abs(float(l_dev) - float(l_ref)) < 3e-2
    for (n, p), (_, q) in zip(ref.named_parameters(), dev.named_parameters()):
        g_ref, g_dev = p.grad, q.grad.float().cpu()
        denom = g_ref.abs().max().item() + 1e-6
        rel = (g_dev - g_ref).abs().max().item() / denom
        assert rel < (0.2 if cfg.precision == "mxfp8" else 8e-2), f"{n}: rel err {rel}"


@pytest.mark.parametrize("precision", ["bf16", "mxfp8"])
def test_trainer_loss_decreases_and_launches_counted(precision):
    cfg = _cfg(head_dim=128, hidden=512, precision=precision)
    tr = PretrainTrainer(cfg, OptimConfig(lr=2e-3), TrainConfig(micro_batch=1, local_batch=2, warmup_steps=1), "cuda")
    toks = synthetic_tokens(1, 2, cfg.seq_len, cfg.vocab_size, seed=0)[0]
    n0 = _lib.launch_count()
    losses = [tr.train_step(toks) for _ in range(6)]
    assert _lib.launch_count() - n0 > 50
    assert losses[-1] < losses[0] - 0.5, losses
    _lib.check_status("trainer")


def test_trainer_masked_labels_match_cpu_trainer():
    """Packed fine-tuning batches: (tokens, labels) with -100 on the unlabelled positions; the mean
    runs over the labelled ones.  GPU trainer against the CPU fp32 trainer from the same weights."""
    cfg = _cfg()
    opt = OptimConfig(lr=1e-3, clip_grad=1.0)
    tc = TrainConfig(micro_batch=1, local_batch=2, warmup_steps=0, seed=2)
    ref = PretrainTrainer(GPTConfig(**{**cfg.to_dict(), "dtype": "fp32"}), opt, tc, "cpu")
    dev = PretrainTrainer(cfg, opt, tc, "cuda")
    with torch.no_grad():
        for (n, p), (_, q) in zip(ref.model.named_parameters(), dev.model.named_parameters()):
            q.copy_(p.to(q.dtype))
            p.copy_(q.float().cpu())
    toks = synthetic_tokens(1, 2, cfg.seq_len, cfg.vocab_size, seed=9, pin=False)[0]
    x, y = toks[:, :-1].contiguous(), toks[:, 1:].clone()
    y[:, :200] = -100
    for _ in range(2):
        a, b = ref.train_step((x, y)), dev.train_step((x, y))
        assert abs(a - b) < 3e-2, (a, b)
    assert abs(ref.engine.grad_norm() - dev.engine.grad_norm()) < 0.1 * ref.engine.grad_norm()
    _lib.check_status("masked trainer")
