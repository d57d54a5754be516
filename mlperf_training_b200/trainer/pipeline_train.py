"""Pre-training steps over a pipeline x data parallel mesh.

``PipelineTrainer`` has the interface of ``trainer.pretrain.PretrainTrainer`` (``train_step``,
``train_step_device``, ``eval_sums``, ``lr``, ``model``, ``engine``, ``n_micro``, ``step_idx``) so the
run loop drives either.  A rank owns one ``parallel.pipeline.GPTStage`` (plain 1F1B) or
``virtual_stages`` of them (interleaved 1F1B); the ranks of one pipeline get the same batch, the
data-parallel replicas of a stage share its ZeRO-sharded optimizer, and the gradient-norm of the
clip is summed over the pipeline group.  With ``tp`` a stage is itself tensor + sequence parallel: the mesh
is tensor x data x pipeline, the ranks of a tensor-parallel group see the same batch and each scores its own
block of token rows.  The loss lives on the last stage and is broadcast to the
pipeline group by an all-reduce, so every rank reports the same number.

The reference reaches this through Megatron's ``get_forward_backward_func`` with
``pipeline_model_parallel_size`` / ``virtual_pipeline_model_parallel_size``
(llama2_sft/primus/src/llama2_custom.py:1494, llama2_sft/primus/conf/llama2_70b_lora_posttrain.yaml:19-21).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ..models.gpt import GPTConfig
from ..parallel.engine import OptimConfig, ZeroEngine, cosine_lr
from ..parallel.pipeline import GPTStage, InterleavedRunner, PipelineRunner, pp_bucket_of
from .pretrain import TrainConfig


def _chunk_bucket_of(name: str) -> str:
    """Parameters of chunk ``c`` of a ``ModuleList`` of stages: bucket per (chunk, block)."""
    c, rest = name.split(".", 1)
    return f"c{int(c):02d}_{pp_bucket_of(rest)}"


class PipelineTrainer:
    def __init__(self, model_cfg: GPTConfig, opt: OptimConfig, train: TrainConfig, device, mesh, virtual_stages: int = 1,
                 freeze_base: bool = False, tp=None, ep_group=None, expert_dp_group=None, cp_group=None, cp_mode: str = "allgather"):
        self.cfg, self.train_cfg = model_cfg, train
        self.device = torch.device(device)
        self.mesh = mesh
        self.S, self.r = mesh.size("pp"), mesh.index("pp")
        self.v = max(int(virtual_stages or 1), 1)
        self.pp_group, self.dp_group = mesh.group("pp"), mesh.group("dp")
        # tensor + sequence parallel stages: the ranks of ``tp.group`` hold slices of one stage and a block of its token rows
        self.tp = tp if (tp is not None and tp.world > 1) else None
        torch.manual_seed(train.seed + 1000 * self.r)       # replicas of a stage start from the same weights
        pp_ranks = mesh.ranks["pp"]
        if self.v == 1:
            self.model = GPTStage(model_cfg, self.r, self.S, device=self.device, tp=self.tp, ep_group=ep_group)
            prev, nxt = mesh.prev_next_stage()
            self.runner = PipelineRunner(self.model, prev, nxt)
            bucket_of = pp_bucket_of
            self.chunks = [self.model]
        else:
            if model_cfg.n_layers < self.S * self.v:
                raise ValueError(f"{model_cfg.n_layers} layers cannot fill {self.S} x {self.v} virtual stages")
            self.chunks = [GPTStage(model_cfg, c * self.S + self.r, self.S * self.v, device=self.device, tp=self.tp, ep_group=ep_group)
                           for c in range(self.v)]
            self.model = nn.ModuleList(self.chunks)
            self.runner = InterleavedRunner(self.chunks, self.r, self.S, pp_ranks[(self.r - 1) % self.S],
                                            pp_ranks[(self.r + 1) % self.S])
            bucket_of = _chunk_bucket_of
        if freeze_base:
            from ..models.lora import freeze_base as _freeze
            _freeze(self.model)
        # context parallel stages: the ranks of ``cp_group`` hold chunks of the same sequences; gradients are reduced
        # over data x context, the loss is the mean of the chunks' losses
        self.cp_group = cp_group if (cp_group is not None and dist.get_world_size(cp_group) > 1) else None
        self.cp_world = dist.get_world_size(self.cp_group) if self.cp_group is not None else 1
        self.cp_rank = dist.get_rank(self.cp_group) if self.cp_group is not None else 0
        self.cp_mode = cp_mode
        if self.cp_group is not None:
            if self.tp is not None:
                raise NotImplementedError("pipeline stages take tensor OR context parallelism")
            for chunk in self.chunks:
                chunk.set_context_parallel(self.cp_group, cp_mode)
        grad_group = mesh.group("dp_cp") if self.cp_group is not None else self.dp_group
        self.engine = ZeroEngine(self.model, opt, group=grad_group, comm="nccl", bucket_of=bucket_of, pp_group=self.pp_group,
                                 tp_group=self.tp.group if self.tp is not None else None, expert_dp_group=expert_dp_group)
        if train.local_batch % train.micro_batch:
            raise ValueError("local_batch must be a multiple of micro_batch")
        self.n_micro = train.local_batch // train.micro_batch
        if self.v > 1 and self.n_micro % self.S:
            raise ValueError(f"interleaved stages need a multiple of {self.S} micro-batches per step, got {self.n_micro}")
        self.step_idx = 0
        self._staging: dict[int, torch.Tensor] = {}
        self.has_loss = self.chunks[-1].last

    def lr(self) -> float:
        o, t = self.engine.opt, self.train_cfg
        return cosine_lr(self.step_idx, base_lr=o.lr, min_lr=o.lr * t.min_lr_ratio, warmup=t.warmup_steps,
                         decay_steps=t.decay_steps)

    @staticmethod
    def _split(tokens, labels):
        if labels is None:
            return tokens[:, :-1].contiguous(), tokens[:, 1:].contiguous()
        return tokens, labels

    def _chunk(self, t: torch.Tensor) -> torch.Tensor:
        """This rank's part of the sequence dimension (everything without context parallelism)."""
        if self.cp_group is None:
            return t
        if self.cp_mode == "ring":
            from ..parallel.context import zigzag_chunk
            return zigzag_chunk(t, self.cp_world, self.cp_rank, dim=1)
        s = t.shape[1] // self.cp_world
        if t.shape[1] % self.cp_world:
            raise ValueError(f"sequence length {t.shape[1]} does not divide over {self.cp_world} context-parallel ranks")
        return t[:, self.cp_rank * s:(self.cp_rank + 1) * s].contiguous()

    def train_step_device(self, tokens: torch.Tensor, labels: torch.Tensor | None = None) -> torch.Tensor:
        """One optimizer step; the mean loss over the micro-batches as a 0-d device tensor on every
        rank of the pipeline."""
        mb = self.train_cfg.micro_batch
        x_all, y_all = self._split(tokens, labels)
        mbs = []
        for i in range(self.n_micro):
            x, y = x_all[i * mb:(i + 1) * mb].contiguous(), y_all[i * mb:(i + 1) * mb].contiguous()
            # explicit labels mask part of the positions (-100): the mean runs over the labelled ones (with the sequence
            # sharded every chunk divides by its share of the count, so the average of the chunks is the mean)
            n_valid = None if labels is None else max(int((y != -100).sum()), 1) / self.cp_world
            x, y = self._chunk(x), self._chunk(y)
            mbs.append((x, y) if labels is None else (x, y, n_valid if self.cp_group is not None else int(n_valid)))
        total = self.runner.run(mbs)
        self.engine.step(self.lr(), grad_scale=1.0 / self.n_micro)
        self.step_idx += 1
        out = torch.zeros((), dtype=torch.float32, device=self.device)
        if total is not None:
            out += total.float() / self.n_micro
        dist.all_reduce(out, group=self.pp_group)
        if self.tp is not None:
            dist.all_reduce(out, group=self.tp.group)          # every rank of a stage scored its own token rows
        if self.cp_group is not None:
            dist.all_reduce(out, group=self.cp_group)
            out = out / self.cp_world
        return out

    def _to_device(self, t: torch.Tensor, slot: int) -> torch.Tensor:
        buf = self._staging.get(slot)
        if buf is None or buf.shape != t.shape:
            buf = self._staging[slot] = torch.empty(t.shape, dtype=torch.int64, device=self.device)
        buf.copy_(t, non_blocking=True)
        return buf

    def train_step(self, batch) -> float:
        if isinstance(batch, (tuple, list)):
            loss = self.train_step_device(self._to_device(batch[0], 0), self._to_device(batch[1], 1))
        else:
            loss = self.train_step_device(self._to_device(batch, 0))
        return float(loss.item())

    @torch.no_grad()
    def eval_sums(self, tokens: torch.Tensor, labels: torch.Tensor | None = None) -> torch.Tensor:
        """Forward-only ``[sum of token losses, labelled tokens]`` summed over every rank's data: each
        micro-batch walks the virtual stages in order (a forward-only pass has no bubble to hide)."""
        mb = self.train_cfg.micro_batch
        x_all, y_all = self._split(tokens, labels)
        acc = torch.zeros(2, dtype=torch.float64, device=self.device)
        pp_ranks = self.mesh.ranks["pp"]
        prev, nxt = pp_ranks[(self.r - 1) % self.S], pp_ranks[(self.r + 1) % self.S]
        for i in range(0, x_all.shape[0], mb):
            x, y = self._chunk(x_all[i:i + mb].contiguous()), self._chunk(y_all[i:i + mb].contiguous())
            tpw = self.tp.world if self.tp is not None else 1
            like = torch.empty((x.numel() // tpw, self.cfg.hidden), dtype=self.cfg.torch_dtype(), device=self.device)
            for chunk in self.chunks:
                act = None
                if not chunk.first:
                    act = torch.empty_like(like)
                    dist.recv(act, src=prev)
                out = chunk(act, x, y, n_valid=1)
                if chunk.last:
                    acc[0] += out.double()
                    rows = y.numel() // tpw                      # this rank scored its own block of token rows
                    mine = y.reshape(-1)[self.tp.rank * rows:(self.tp.rank + 1) * rows] if self.tp is not None else y
                    acc[1] += (mine != -100).sum().double()
                else:
                    dist.send(out.contiguous(), dst=nxt)
        dist.all_reduce(acc, group=self.pp_group)        # only the last stage contributed
        if self.tp is not None:
            dist.all_reduce(acc, group=self.tp.group)
        if self.cp_group is not None:
            dist.all_reduce(acc, group=self.cp_group)      # sums and counts of the chunks
        if dist.get_world_size(self.dp_group) > 1:
            dist.all_reduce(acc, group=self.dp_group)
        return acc

    @torch.no_grad()
    def eval_loss(self, tokens: torch.Tensor, labels: torch.Tensor | None = None) -> torch.Tensor:
        s = self.eval_sums(tokens, labels)
        return (s[0] / s[1].clamp(min=1)).float()
