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
every shipped config sets the size to 1.  Interleaved (virtual) stages are accepted as a knob and
run as the plain schedule (one model chunk per rank).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ..models.gpt import Block, GPTConfig
from ..ops import functional as F
from ..ops import kernels as K


def stage_layers(n_layers: int, n_stages: int, stage: int) -> range:
    """Contiguous, as even as possible; earlier stages take the remainder."""
    base, rem = divmod(n_layers, n_stages)
    lo = stage * base + min(stage, rem)
    return range(lo, lo + base + (1 if stage < rem else 0))


class GPTStage(nn.Module):
    def __init__(self, cfg: GPTConfig, stage: int, n_stages: int, device="cpu", tp=None):
        super().__init__()
        self.cfg, self.stage, self.n_stages = cfg, stage, n_stages
        self.first, self.last = stage == 0, stage == n_stages - 1
        self.layers = stage_layers(cfg.n_layers, n_stages, stage)
        dtype = cfg.torch_dtype()
        if self.first:
            self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden, dtype=dtype, device=device))
        self.blocks = nn.ModuleList([Block(cfg, i, dtype, device, tp=tp) for i in self.layers])
        if self.last:
            self.final_norm = nn.Parameter(torch.ones(cfg.hidden, dtype=dtype, device=device))
            self.lm_head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden, dtype=dtype, device=device))
        self._rope = None
        with torch.no_grad():
            for n, p in self.named_parameters():
                if p.dim() >= 2 and "lora" not in n:
                    p.normal_(0.0, cfg.init_std)

    @torch.no_grad()
    def load_from_full(self, full: nn.Module) -> None:
        """Copy this stage's parameters out of an unsplit ``models.gpt.GPT``."""
        if self.first:
            self.embed.copy_(full.embed)
        for blk, i in zip(self.blocks, self.layers):
            blk.load_state_dict(full.blocks[i].state_dict())
        if self.last:
            self.final_norm.copy_(full.final_norm)
            self.lm_head.copy_(full.lm_head)

    def rope(self, device):
        if self._rope is None or self._rope[0].device != torch.device(device):
            self._rope = K.rope_tables(self.cfg.seq_len, self.cfg.head_dim, self.cfg.rope_theta, device)
        return self._rope

    def forward(self, x, tokens: torch.Tensor, labels: torch.Tensor | None):
        """``x``: incoming activation ``[B*S, hidden]`` (ignored on the first stage, which embeds
        ``tokens``).  Returns the outgoing activation, or the mean loss on the last stage."""
        B, S = tokens.shape
        cos, sin = self.rope(tokens.device)
        if self.first:
            x = F.embedding(tokens.reshape(-1), self.embed)
        for blk in self.blocks:
            x = blk(x, cos, sin, B, S)
        if self.last:
            return F.lm_head_loss(x, self.final_norm, self.lm_head, labels.reshape(-1), eps=self.cfg.norm_eps,
                                  precision=self.cfg.precision)
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
        act_like = torch.empty((tok0.numel(), st.cfg.hidden), dtype=st.cfg.torch_dtype(), device=tok0.device)
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
