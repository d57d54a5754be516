"""Pipeline parallelism: a GPT split into contiguous layer ranges (stages) and the 1F1B schedule
over point-to-point messages.

Each stage owns ``n_layers / n_stages`` transformer blocks (the first also the embedding, the last
the final norm, the vocabulary projection and the loss).  A step runs ``M`` micro-batches through the
non-interleaved one-forward-one-backward schedule: ``S - s - 1`` warm-up forwards on stage ``s``, then
forward/backward pairs, then the remaining backwards, so at most ``S - s`` activations are alive on a
stage.  Activations ``[tokens, hidden]`` and their gradients travel with ``torch.distributed`` p2p ops
(NCCL ``isend`` / ``irecv`` on GPUs, gloo on CPU), paired in one ``batch_isend_irecv`` whenever a stage
both sends and receives, which is what keeps neighbouring stages from blocking each other.

The reference gets this schedule from Megatron's ``get_forward_backward_func``
(llama2_sft/primus/src/llama2_custom.py:1494) with ``pipeline_model_parallel_size`` /
``virtual_pipeline_model_parallel_size`` from the YAML (llama2_sft/primus/conf/llama2_70b_lora_posttrain.yaml:19-21);
every shipped config sets the size to 1.  A stage may itself be tensor + sequence parallel (``tp``): its ranks
then hold slices of the stage's matrices, each passes its own block of token rows to the same-index rank of
the next stage, and the messages shrink by the group size.  With ``ep_group`` the experts of a stage's
mixture-of-experts blocks are spread over the data-parallel replicas of the stage, which follow the same
schedule and so meet in the same token exchanges.  ``InterleavedRunner`` is the virtual-stage variant (several
model chunks per rank); ``trainer.pipeline_train.PipelineTrainer`` puts either schedule behind the
trainer interface of the run loop.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ..models.gpt import Block, GPTConfig, shard_of
from ..ops import functional as F
from ..ops import kernels as K


def stage_layers(n_layers: int, n_stages: int, stage: int) -> range:
    """Contiguous, as even as possible; earlier stages take the remainder."""
    base, rem = divmod(n_layers, n_stages)
    lo = stage * base + min(stage, rem)
    return range(lo, lo + base + (1 if stage < rem else 0))


class GPTStage(nn.Module):
    def __init__(self, cfg: GPTConfig, stage: int, n_stages: int, device="cpu", tp=None, ep_group=None):
        super().__init__()
        self.cfg, self.stage, self.n_stages = cfg, stage, n_stages
        self.first, self.last = stage == 0, stage == n_stages - 1
        self.layers = stage_layers(cfg.n_layers, n_stages, stage)
        dtype = cfg.torch_dtype()
        if self.first:
            self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden, dtype=dtype, device=device))
        self.blocks = nn.ModuleList([Block(cfg, i, dtype, device, tp=tp, ep_group=ep_group) for i in self.layers])
        if self.last:
            self.final_norm = nn.Parameter(torch.ones(cfg.hidden, dtype=dtype, device=device))
            self.lm_head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden, dtype=dtype, device=device))
        self._rope = None
        self.tp = tp if (tp is not None and tp.world > 1) else None
        with torch.no_grad():
            for n, p in self.named_parameters():
                if p.dim() >= 2 and "lora" not in n:
                    shard = getattr(p, "tensor_parallel", None)
                    if shard is None:
                        p.normal_(0.0, cfg.init_std)
                        continue
                    # tensor-parallel slice: draw the full matrix (the ranks of a stage share the seed, so they draw
                    # the same one) and keep this rank's part - equal slices would never grow apart
                    kind, W, r = shard
                    full_shape = (p.shape[0] * W, p.shape[1]) if kind in ("rows", "rows_2", "qkv") else (p.shape[0], p.shape[1] * W)
                    full = torch.empty(full_shape, dtype=p.dtype, device=p.device).normal_(0.0, cfg.init_std)
                    p.copy_(shard_of(full, kind, W, r, cfg))

    @torch.no_grad()
    def load_from_full(self, full: nn.Module) -> None:
        """Copy this stage's parameters out of an unsplit ``models.gpt.GPT``."""
        if self.first:
            self.embed.copy_(full.embed)
        for blk, i in zip(self.blocks, self.layers):
            src = dict(full.blocks[i].named_parameters())
            for n, p in blk.named_parameters():
                shard = getattr(p, "tensor_parallel", None)
                if shard is not None and src[n].shape != p.shape:        # the unsplit model holds the whole matrix
                    p.copy_(shard_of(src[n], shard[0], shard[1], shard[2], self.cfg))
                elif getattr(p, "expert_parallel", False) and src[n].shape != p.shape:
                    ep, ep_rank = p.expert_shard                         # this rank's block of the stacked experts
                    per = src[n].shape[0] // ep
                    p.copy_(src[n][ep_rank * per:(ep_rank + 1) * per])
                else:
                    p.copy_(src[n])
        if self.last:
            self.final_norm.copy_(full.final_norm)
            self.lm_head.copy_(full.lm_head)

    def set_context_parallel(self, group, mode: str = "allgather") -> None:
        """Shard the sequence over ``group`` inside this stage: ``forward`` then takes the rank's chunk of tokens and
        labels (chunk ``r`` of ``W``; with ``mode="ring"`` the zig-zag chunks ``r`` and ``2 W - 1 - r``) - see
        ``models.gpt.GPT.set_context_parallel``."""
        if group is None or dist.get_world_size(group) == 1:
            self.cp = None
            for blk in self.blocks:
                blk.cp = None
            return
        if self.cfg.sink:
            raise NotImplementedError("context parallelism does not carry attention sink logits")
        if mode not in ("allgather", "ulysses", "ring"):
            raise ValueError(f"unknown context-parallel mode '{mode}'")
        self.cp = (group, dist.get_world_size(group), dist.get_rank(group), mode)
        for blk in self.blocks:
            blk.cp = (group, mode)

    def rope(self, device):
        if self._rope is None or self._rope[0].device != torch.device(device):
            self._rope = K.rope_tables(self.cfg.seq_len, self.cfg.head_dim, self.cfg.rope_theta, device)
        return self._rope

    def forward(self, x, tokens: torch.Tensor, labels: torch.Tensor | None, n_valid=None):
        """``x``: incoming activation ``[B*S, hidden]`` (ignored on the first stage, which embeds
        ``tokens``).  Returns the outgoing activation, or the mean loss on the last stage (the sum of
        the token losses divided by ``n_valid`` when that is given)."""
        B, S = tokens.shape
        cos, sin = self.rope(tokens.device)
        if getattr(self, "cp", None) is not None:
            _, W, r, mode = self.cp
            if mode == "ring":
                from .context import zigzag_chunk
                cos, sin = zigzag_chunk(cos[:S * W], W, r, dim=0), zigzag_chunk(sin[:S * W], W, r, dim=0)
            else:
                cos, sin = cos[r * S:(r + 1) * S].contiguous(), sin[r * S:(r + 1) * S].contiguous()
        ids = tokens.reshape(-1)
        if self.tp is not None:
            # tensor + sequence parallel inside the stage: every rank of the group embeds, passes on and scores its
            # own block of token rows; the returned loss is this rank's share of the mean
            W, r = self.tp.world, self.tp.rank
            if ids.numel() % W:
                raise ValueError("the number of tokens must be divisible by the tensor-parallel size")
            rows = ids.numel() // W
            if n_valid is None:
                n_valid = ids.numel()
            ids = ids[r * rows:(r + 1) * rows]
            if labels is not None:
                labels = labels.reshape(-1)[r * rows:(r + 1) * rows]
        if self.first:
            x = F.embedding(ids, self.embed)
        for blk in self.blocks:
            x = blk(x, cos, sin, B, S)
        if self.last:
            return F.lm_head_loss(x, self.final_norm, self.lm_head, labels.reshape(-1), eps=self.cfg.norm_eps,
                                  n_valid=n_valid, precision=self.cfg.precision)
        return x


def pp_bucket_of(name: str) -> str:
    parts = name.split(".")
    if parts[0] == "blocks":
        return f"block{int(parts[1]):04d}"
    return "a_embed" if parts[0] == "embed" else "z_head"


class PipelineRunner:
    """Drives one stage.  ``prev_rank`` / ``next_rank`` are global ranks (None at the ends)."""

    def __init__(self, stage: GPTStage, prev_rank: int | None, next_rank: int | None, group=None):
        self.stage, self.prev, self.next, self.group = stage, prev_rank, next_rank, group

    # ------------------------------------------------------------------ p2p
    def _exchange(self, send_next=None, send_prev=None, recv_prev_like=None, recv_next_like=None):
        ops, got_prev, got_next = [], None, None
        if send_next is not None and self.next is not None:
            ops.append(dist.P2POp(dist.isend, send_next.contiguous(), self.next, self.group))
        if send_prev is not None and self.prev is not None:
            ops.append(dist.P2POp(dist.isend, send_prev.contiguous(), self.prev, self.group))
        if recv_prev_like is not None and self.prev is not None:
            got_prev = torch.empty_like(recv_prev_like)
            ops.append(dist.P2POp(dist.irecv, got_prev, self.prev, self.group))
        if recv_next_like is not None and self.next is not None:
            got_next = torch.empty_like(recv_next_like)
            ops.append(dist.P2POp(dist.irecv, got_next, self.next, self.group))
        if ops:
            for r in dist.batch_isend_irecv(ops):
                r.wait()
        return got_prev, got_next

    # ------------------------------------------------------------------ one step
    def run(self, micro_batches: list[tuple[torch.Tensor, torch.Tensor]]) -> torch.Tensor | None:
        """Forward + backward of all micro-batches ``(tokens [b,S], labels [b,S])`` in 1F1B order.
        Gradients are left in ``main_grad`` / ``.grad`` (scale by ``1 / len(micro_batches)`` in the
        optimizer step).  Returns the summed loss on the last stage, None elsewhere."""
        st = self.stage
        M = len(micro_batches)
        S, s = st.n_stages, st.stage
        tok0 = micro_batches[0][0]
        act_like = torch.empty((tok0.numel() // (st.tp.world if st.tp is not None else 1), st.cfg.hidden),
                               dtype=st.cfg.torch_dtype(), device=tok0.device)
        warm = min(S - s - 1, M)
        steady = M - warm
        live: list[tuple[torch.Tensor | None, torch.Tensor]] = []
        total = None

        def fwd(i, x):
            if x is not None:
                x.requires_grad_(True)
            out = st(x, *micro_batches[i])
            live.append((x, out))
            return out

        def bwd(grad):
            nonlocal total
            x, out = live.pop(0)
            if st.last:
                out.backward()
                total = out.detach() if total is None else total + out.detach()
            else:
                torch.autograd.backward(out, grad)
            return None if x is None else x.grad

        x = None
        for i in range(warm):
            if not st.first:
                x, _ = self._exchange(recv_prev_like=act_like)
            out = fwd(i, x)
            self._exchange(send_next=out.detach())
        if steady > 0 and not st.first:
            x, _ = self._exchange(recv_prev_like=act_like)
        for i in range(steady):
            out = fwd(warm + i, x)
            grad = None
            if not st.last:
                _, grad = self._exchange(send_next=out.detach(), recv_next_like=act_like)
            gin = bwd(grad)
            if i + 1 < steady:
                x, _ = self._exchange(send_prev=gin, recv_prev_like=act_like if not st.first else None)
            else:
                self._exchange(send_prev=gin)
        for _ in range(warm):
            _, grad = self._exchange(recv_next_like=act_like)
            gin = bwd(grad)
            self._exchange(send_prev=gin)
        return total


class InterleavedRunner:
    """Interleaved (virtual-stage) 1F1B: every rank owns ``v`` model chunks; chunk ``c`` of rank ``r``
    is virtual stage ``c * S + r`` of ``S * v``.  Micro-batches advance through the virtual stages in
    groups of ``S``; a rank runs ``(S - r - 1) * 2 + (v - 1) * S`` warm-up forwards, then alternates
    one forward with one backward, then drains the backwards - the schedule Megatron uses for
    ``virtual_pipeline_model_parallel_size`` (llama2_sft/primus/conf/llama2_70b_lora_posttrain.yaml:21,
    null in every shipped configuration).  The pipeline bubble shrinks by the factor ``v`` against the
    plain schedule at the price of ``v`` times more messages.  The number of micro-batches must be a
    multiple of ``S``.  Messages go to the ring neighbours (the last rank's output feeds the first
    rank's next chunk); whenever a rank sends and receives at one point of the schedule the operations
    are posted together in one ``batch_isend_irecv``."""

    def __init__(self, chunks: list[GPTStage], rank: int, n_ranks: int, prev_rank: int, next_rank: int, group=None):
        self.chunks, self.r, self.S, self.v = chunks, rank, n_ranks, len(chunks)
        self.prev, self.next, self.group = prev_rank, next_rank, group

    def _exchange(self, send_next=None, send_prev=None, recv_prev=None, recv_next=None):
        ops, got_prev, got_next = [], None, None
        if send_next is not None:
            ops.append(dist.P2POp(dist.isend, send_next.contiguous(), self.next, self.group))
        if send_prev is not None:
            ops.append(dist.P2POp(dist.isend, send_prev.contiguous(), self.prev, self.group))
        if recv_prev is not None:
            got_prev = torch.empty_like(recv_prev)
            ops.append(dist.P2POp(dist.irecv, got_prev, self.prev, self.group))
        if recv_next is not None:
            got_next = torch.empty_like(recv_next)
            ops.append(dist.P2POp(dist.irecv, got_next, self.next, self.group))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        return got_prev, got_next

    def run(self, micro_batches: list[tuple[torch.Tensor, torch.Tensor]]) -> torch.Tensor | None:
        S, v, r = self.S, self.v, self.r
        M = len(micro_batches)
        if M % S:
            raise ValueError(f"{M} micro-batches are not a multiple of the {S} pipeline ranks")
        total = M * v
        warm = min((S - r - 1) * 2 + (v - 1) * S, total)
        remain = total - warm
        cfg = self.chunks[0].cfg
        tok0 = micro_batches[0][0]
        tp = self.chunks[0].tp
        like = torch.empty((tok0.numel() // (tp.world if tp is not None else 1), cfg.hidden), dtype=cfg.torch_dtype(),
                           device=tok0.device)
        inputs = [[] for _ in range(v)]
        outputs = [[] for _ in range(v)]
        ograds = [[] for _ in range(v)]
        loss_sum = None

        def chunk_of(k, fwd=True):
            c = (k % (S * v)) // S
            return c if fwd else v - 1 - c

        def mb_of(k):
            return (k // (S * v)) * S + k % S

        def is_first(c):
            return r == 0 and c == 0

        def is_last(c):
            return r == S - 1 and c == v - 1

        def fwd(k):
            c = chunk_of(k)
            if is_first(c) and len(inputs[c]) == len(outputs[c]):
                inputs[c].append(None)
            x = inputs[c][len(outputs[c])]
            if x is not None:
                x.requires_grad_(True)
            out = self.chunks[c](x, *micro_batches[mb_of(k)])
            outputs[c].append(out)
            return None if is_last(c) else out.detach()

        def bwd(k):
            nonlocal loss_sum
            c = chunk_of(k, False)
            x, out = inputs[c].pop(0), outputs[c].pop(0)
            if is_last(c):
                out.backward()
                loss_sum = out.detach() if loss_sum is None else loss_sum + out.detach()
            else:
                torch.autograd.backward(out, ograds[c].pop(0))
            return None if (x is None or is_first(c)) else x.grad

        def want_prev(k_next):                     # does forward step k_next take its input from a message?
            return k_next < total and not is_first(chunk_of(k_next))

        def want_next(k_next):                     # does backward step k_next take its gradient from a message?
            return k_next < total and not is_last(chunk_of(k_next, False))

        # the input of the very first forward
        if want_prev(0):
            x, _ = self._exchange(recv_prev=like)
            inputs[chunk_of(0)].append(x)
        for k in range(warm):
            out = fwd(k)
            rp = like if want_prev(k + 1) else None
            rn = like if (k == warm - 1 and remain > 0 and want_next(0)) else None
            x, g = self._exchange(send_next=out, recv_prev=rp, recv_next=rn)
            if rp is not None:
                inputs[chunk_of(k + 1)].append(x)
            if rn is not None:
                ograds[chunk_of(0, False)].append(g)
        if remain == 0 and want_next(0):
            _, g = self._exchange(recv_next=like)
            ograds[chunk_of(0, False)].append(g)
        for k in range(remain):
            fk, bk = k + warm, k
            out = fwd(fk)
            gin = bwd(bk)
            rp = like if want_prev(fk + 1) else None
            rn = like if want_next(bk + 1) else None
            x, g = self._exchange(send_next=out, send_prev=gin, recv_prev=rp, recv_next=rn)
            if rp is not None:
                inputs[chunk_of(fk + 1)].append(x)
            if rn is not None:
                ograds[chunk_of(bk + 1, False)].append(g)
        for bk in range(remain, total):
            gin = bwd(bk)
            rn = like if want_next(bk + 1) else None
            _, g = self._exchange(send_prev=gin, recv_next=rn)
            if rn is not None:
                ograds[chunk_of(bk + 1, False)].append(g)
        return loss_sum
