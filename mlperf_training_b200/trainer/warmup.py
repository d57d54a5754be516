"""Synthetic warm-up before ``run_start`` with exact state restoration.

Running a few real training steps on random tokens before the timed region loads every kernel,
sizes the allocator pools and fills caches; afterwards the model must be indistinguishable from a
freshly initialised one.  The sequence is the reference's
(primus_mllog/warmup.py:584-738 in the bundled wheel; SFT variant with forward-only validation
warm-up in llama2_sft/primus/src/llama2_custom.py:1059-1292):

1. snapshot parameters (to CPU), optimizer moments and step counter, LR-schedule position;
2. run N ``train_step`` calls on random tokens (and optionally M forward-only evaluation steps);
3. restore parameters, zero the Adam moments and gradients, reset step counters, drop cached
   low-precision weight copies and any per-site scale state, empty the allocator cache, barrier.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops.linear import bump_weight_epoch


def snapshot_engine(engine) -> dict:
    return {
        "params": [b.param_buf.detach().to("cpu", copy=True) for b in engine.buckets],
        "master": [None if b.master is None else b.master.detach().to("cpu", copy=True) for b in engine.buckets],
        "step": engine.step_count,
    }


def restore_engine(engine, snap: dict) -> None:
    with torch.no_grad():
        for b, p, mw in zip(engine.buckets, snap["params"], snap["master"]):
            b.param_buf.copy_(p.to(b.param_buf.device))
            b.grad_buf.zero_()
            b.m.zero_()
            b.v.zero_()
            if b.master is not None and mw is not None:
                b.master.copy_(mw.to(b.master.device))
    engine.step_count = snap["step"]
    engine.last_grad_norm = None
    bump_weight_epoch()


def run_synthetic_warmup(trainer, train_steps: int = 2, eval_steps: int = 0, seed: int = 1234) -> dict:
    """Warm up ``trainer`` (a ``PretrainTrainer``-like object with ``engine``, ``cfg``,
    ``train_cfg``, ``train_step_device``, ``eval_loss``, ``step_idx``) and restore its state.
    Returns a small report (losses seen, for logging only)."""
    if train_steps <= 0 and eval_steps <= 0:
        return {"train_losses": [], "eval_losses": []}
    engine = trainer.engine
    snap = snapshot_engine(engine)
    step_idx = trainer.step_idx
    dev = trainer.device
    gen = torch.Generator(device="cpu").manual_seed(seed)
    lb, S, V = trainer.train_cfg.local_batch, trainer.cfg.seq_len, trainer.cfg.vocab_size
    report = {"train_losses": [], "eval_losses": []}
    rng_state = torch.get_rng_state()
    cuda_state = torch.cuda.get_rng_state(dev) if dev.type == "cuda" else None
    for _ in range(train_steps):
        toks = torch.randint(0, V, (lb, S + 1), generator=gen).to(dev)
        report["train_losses"].append(float(trainer.train_step_device(toks)))
    for _ in range(eval_steps):
        toks = torch.randint(0, V, (trainer.train_cfg.micro_batch, S + 1), generator=gen).to(dev)
        report["eval_losses"].append(float(trainer.eval_loss(toks)))
    restore_engine(engine, snap)
    trainer.step_idx = step_idx
    torch.set_rng_state(rng_state)
    if cuda_state is not None:
        torch.cuda.set_rng_state(cuda_state, dev)
        torch.cuda.empty_cache()
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
    return report
