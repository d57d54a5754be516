"""Pre-training step loop for the GPT family: micro-batching with gradient accumulation,
LR schedule, sharded optimizer step, loss reporting.

``PretrainTrainer.train_step(batch)`` is the public call a user makes: it takes one global
step's token ids for this rank from (pinned) host memory, copies them to the device, runs
forward / backward over the micro-batches, applies the optimizer and returns the mean loss as a
Python float.  ``train_step_device`` is the same step on tokens already resident on the device
and returns the loss as a device tensor (no host synchronisation), which is what the
device-timed benchmark loop uses.

Mirrors the step structure of the reference's Megatron trainer as wrapped by
``MLPerfMegatronPretrainTrainer.train_step`` (primus_mllog/mlperf_pre_training.py:243-262 in the
bundled wheel): ``forward_backward_func`` over GBS / (MBS * DP) micro-batches, then
``optimizer.step``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..models.gpt import GPT, GPTConfig
from ..parallel.engine import OptimConfig, ZeroEngine, cosine_lr


@dataclass
class TrainConfig:
    micro_batch: int = 1            # sequences per micro-batch per rank
    local_batch: int = 4            # sequences per step per rank (global batch / data-parallel size)
    warmup_steps: int = 64
    decay_steps: int = 1_200_000
    min_lr_ratio: float = 0.1
    seed: int = 0
    comm: str = "nccl"


class PretrainTrainer:
    def __init__(self, model_cfg: GPTConfig, opt: OptimConfig, train: TrainConfig, device, group=None, ep_group=None):
        self.cfg = model_cfg
        self.train_cfg = train
        self.device = torch.device(device)
        self.model = GPT(model_cfg, device=self.device, seed=train.seed, ep_group=ep_group)
        self.engine = ZeroEngine(self.model, opt, group=group, comm=train.comm)
        self.step_idx = 0
        if train.local_batch % train.micro_batch != 0:
            raise ValueError("local_batch must be a multiple of micro_batch")
        self.n_micro = train.local_batch // train.micro_batch
        self._staging = None

    def lr(self) -> float:
        o, t = self.engine.opt, self.train_cfg
        return cosine_lr(self.step_idx, base_lr=o.lr, min_lr=o.lr * t.min_lr_ratio, warmup=t.warmup_steps,
                         decay_steps=t.decay_steps)

    def train_step_device(self, tokens: torch.Tensor) -> torch.Tensor:
        """``tokens``: int64 ``[local_batch, seq_len + 1]`` on the device.  Returns the mean loss
        over the step's micro-batches as a 0-d device tensor."""
        mb = self.train_cfg.micro_batch
        total = None
        for i in range(self.n_micro):
            chunk = tokens[i * mb:(i + 1) * mb]
            loss = self.model(chunk[:, :-1], chunk[:, 1:])
            loss.backward()
            d = loss.detach()
            total = d if total is None else total + d
        self.engine.step(self.lr(), grad_scale=1.0 / self.n_micro)
        self.step_idx += 1
        return total / self.n_micro

    def train_step(self, batch: torch.Tensor) -> float:
        """One optimizer step from host token ids ``[local_batch, seq_len + 1]`` (int64, ideally
        pinned).  Host -> device copy, step, and a device -> host read of the loss."""
        if self._staging is None or self._staging.shape != batch.shape:
            self._staging = torch.empty(batch.shape, dtype=torch.int64, device=self.device)
        self._staging.copy_(batch, non_blocking=True)
        loss = self.train_step_device(self._staging)
        return float(loss.item())

    @torch.no_grad()
    def eval_loss(self, tokens: torch.Tensor) -> torch.Tensor:
        """Forward-only mean loss on device tokens ``[b, seq_len + 1]``."""
        mb = self.train_cfg.micro_batch
        tot, n = None, 0
        for i in range(0, tokens.shape[0], mb):
            chunk = tokens[i:i + mb]
            l = self.model(chunk[:, :-1], chunk[:, 1:])
            tot = l if tot is None else tot + l
            n += 1
        tot = tot / n
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(tot, op=dist.ReduceOp.AVG)
        return tot


def synthetic_tokens(steps: int, local_batch: int, seq_len: int, vocab: int, seed: int, rank: int = 0,
                     pin: bool = True) -> torch.Tensor:
    """Uniform token ids ``[steps, local_batch, seq_len + 1]`` (int64) from ``seed`` (and rank),
    in pinned host memory when CUDA is present: the synthetic stand-in for the C4 stream
    (the reference's warm-up uses the same kind of random batch, primus_mllog/warmup.py:80-108)."""
    g = torch.Generator().manual_seed(seed * 1000003 + rank)
    t = torch.randint(0, vocab, (steps, local_batch, seq_len + 1), generator=g, dtype=torch.int64)
    if pin and torch.cuda.is_available():
        t = t.pin_memory()
    return t
