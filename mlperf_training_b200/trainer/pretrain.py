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
    zero_stage: int = 1             # 1: optimizer state sharded, parameters replicated; 3: block matrices sharded too


class PretrainTrainer:
    """``group`` is the data-parallel group, ``tp`` an optional ``parallel.tensor.TPContext`` (the
    ranks of one tensor-parallel group must be fed the same batch).  With ``cp_group`` the sequence is
    sharded over that group: its ranks are fed the same batch, each keeps its chunk of every
    sequence, and ``group`` must then span data x context ranks (parameters are replicated over both)."""

    def __init__(self, model_cfg: GPTConfig, opt: OptimConfig, train: TrainConfig, device, group=None, ep_group=None,
                 tp=None, freeze_base: bool = False, replicate_group=None, cp_group=None, cp_mode: str = "allgather",
                 expert_dp_group=None):
        self.cfg = model_cfg
        self.train_cfg = train
        self.device = torch.device(device)
        self.tp = tp if (tp is not None and tp.world > 1) else None
        self.model = GPT(model_cfg, device=self.device, seed=train.seed, ep_group=ep_group, tp=self.tp)
        if freeze_base:
            from ..models.lora import freeze_base as _freeze
            _freeze(self.model)
        if int(train.zero_stage) == 3:
            if self.tp is not None or ep_group is not None or replicate_group is not None or cp_group is not None:
                raise NotImplementedError("zero_stage 3 shards the block matrices over plain data-parallel ranks "
                                          "(no tensor / expert / context parallelism, no hybrid sharding)")
            from ..parallel.zero3 import Zero3Engine
            self.engine = Zero3Engine(self.model, opt, group=group, comm=train.comm)
        else:
            self.engine = ZeroEngine(self.model, opt, group=group, comm=train.comm,
                                     tp_group=self.tp.group if self.tp is not None else None, replicate_group=replicate_group,
                                     expert_dp_group=expert_dp_group)
        self.cp_group = cp_group if (cp_group is not None and dist.get_world_size(cp_group) > 1) else None
        self.cp_world = dist.get_world_size(self.cp_group) if self.cp_group is not None else 1
        self.cp_rank = dist.get_rank(self.cp_group) if self.cp_group is not None else 0
        self.cp_mode = cp_mode
        if self.cp_group is not None:
            self.model.set_context_parallel(self.cp_group, cp_mode)
        self.dp_group = group
        self.replicate_group = replicate_group
        self.step_idx = 0
        if train.local_batch % train.micro_batch != 0:
            raise ValueError("local_batch must be a multiple of micro_batch")
        self.n_micro = train.local_batch // train.micro_batch
        self._staging = None
        self._masked = False
        self.overlap_grad_reduce = True

    def lr(self) -> float:
        o, t = self.engine.opt, self.train_cfg
        return cosine_lr(self.step_idx, base_lr=o.lr, min_lr=o.lr * t.min_lr_ratio, warmup=t.warmup_steps,
                         decay_steps=t.decay_steps)

    def _split(self, tokens: torch.Tensor, labels: torch.Tensor | None):
        """``[b, S+1]`` token rows -> (inputs, labels); explicit ``labels [b, S]`` go with ``tokens [b, S]``."""
        if labels is None:
            return tokens[:, :-1], tokens[:, 1:]
        return tokens, labels

    def _chunk(self, t: torch.Tensor) -> torch.Tensor:
        """This rank's part of the sequence dimension (everything without context parallelism)."""
        if self.cp_group is None:
            return t
        s = t.shape[1] // self.cp_world
        if t.shape[1] % self.cp_world:
            raise ValueError(f"sequence length {t.shape[1]} does not divide over {self.cp_world} context-parallel ranks")
        if self.cp_mode == "ring":
            from ..parallel.context import zigzag_chunk
            return zigzag_chunk(t, self.cp_world, self.cp_rank, dim=1)
        return t[:, self.cp_rank * s:(self.cp_rank + 1) * s].contiguous()

    def _loss(self, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        # explicit labels mask part of the positions (-100): the mean runs over the labelled ones.  With the
        # sequence sharded, every chunk divides by its share of the count, so that the average of the chunks'
        # losses (which is what the gradient reduction forms) is the mean over the whole sequence.
        masked = self._masked
        n_valid = max(int((y != -100).sum()), 1) / self.cp_world if masked else None
        if n_valid is not None and self.cp_group is None:
            n_valid = int(n_valid)
        loss = self.model(self._chunk(x), self._chunk(y), n_valid=n_valid)
        return loss

    def train_step_device(self, tokens: torch.Tensor, labels: torch.Tensor | None = None) -> torch.Tensor:
        """``tokens``: int64 ``[local_batch, seq_len + 1]`` on the device (or ``[local_batch, seq_len]``
        with explicit ``labels``, -100 = no loss).  Returns the mean loss over the step's micro-batches
        as a 0-d device tensor (summed over the tensor-parallel group when there is one)."""
        mb = self.train_cfg.micro_batch
        self._masked = labels is not None
        x_all, y_all = self._split(tokens, labels)
        total = None
        for i in range(self.n_micro):
            last = i == self.n_micro - 1
            if last and self.overlap_grad_reduce:
                # reduce every block's gradients while the rest of this backward still runs
                self.engine.begin_overlap()
                self.model.grad_ready_hook = self.engine.on_block_grads_ready
            loss = self._loss(x_all[i * mb:(i + 1) * mb], y_all[i * mb:(i + 1) * mb])
            loss.backward()
            self.model.grad_ready_hook = None
            d = loss.detach()
            total = d if total is None else total + d
        self.engine.step(self.lr(), grad_scale=1.0 / self.n_micro)
        self.step_idx += 1
        total = total / self.n_micro
        if self.tp is not None:
            total = self.tp.all_reduce(total.float().clone())
        if self.cp_group is not None:
            total = total.float().clone()
            dist.all_reduce(total, group=self.cp_group)
            total = total / self.cp_world
        return total

    def _to_device(self, t: torch.Tensor, slot: int) -> torch.Tensor:
        if self._staging is None:
            self._staging = {}
        buf = self._staging.get(slot)
        if buf is None or buf.shape != t.shape:
            buf = self._staging[slot] = torch.empty(t.shape, dtype=torch.int64, device=self.device)
        buf.copy_(t, non_blocking=True)
        return buf

    def train_step(self, batch) -> float:
        """One optimizer step from host token ids ``[local_batch, seq_len + 1]`` (int64, ideally
        pinned), or a ``(tokens, labels)`` pair of ``[local_batch, seq_len]`` tensors for packed
        fine-tuning data.  Host -> device copy, step, and a device -> host read of the loss."""
        if isinstance(batch, (tuple, list)):
            loss = self.train_step_device(self._to_device(batch[0], 0), self._to_device(batch[1], 1))
        else:
            loss = self.train_step_device(self._to_device(batch, 0))
        return float(loss.item())

    @torch.no_grad()
    def eval_sums(self, tokens: torch.Tensor, labels: torch.Tensor | None = None) -> torch.Tensor:
        """Forward-only ``[sum of token losses, number of labelled tokens]`` on device tokens, summed
        over every rank: evaluation averages over tokens, not over micro-batches (the reference
        accumulates the same pair, llama2_sft/primus/src/llama2_custom.py:752-915)."""
        mb = self.train_cfg.micro_batch
        x_all, y_all = self._split(tokens, labels)
        acc = torch.zeros(2, dtype=torch.float64, device=self.device)
        for i in range(0, x_all.shape[0], mb):
            x, y = self._chunk(x_all[i:i + mb]), self._chunk(y_all[i:i + mb])
            n = (y != -100).sum()
            l = self.model(x, y, n_valid=1)            # n_valid = 1: the plain sum of token losses
            if self.tp is not None:
                l = self.tp.all_reduce(l.float().clone())
            acc[0] += l.double()
            acc[1] += n.double()
        if dist.is_available() and dist.is_initialized():
            g = self.dp_group
            if g is not None:
                if dist.get_world_size(g) > 1:
                    dist.all_reduce(acc, group=g)
            elif self.tp is None and dist.get_world_size() > 1:
                dist.all_reduce(acc)
            if self.replicate_group is not None and dist.get_world_size(self.replicate_group) > 1:
                dist.all_reduce(acc, group=self.replicate_group)      # every rank must see the same evaluation result
        return acc

    @torch.no_grad()
    def eval_loss(self, tokens: torch.Tensor, labels: torch.Tensor | None = None) -> torch.Tensor:
        """Forward-only token-mean loss on device tokens ``[b, seq_len + 1]``."""
        s = self.eval_sums(tokens, labels)
        return (s[0] / s[1].clamp(min=1)).float()


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
