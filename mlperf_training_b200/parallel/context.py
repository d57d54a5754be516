"""Context parallelism: the sequence is cut into ``W`` contiguous chunks, rank ``r`` holds the
queries, keys and values of chunk ``r``.

Causal attention of chunk ``r`` needs the keys and values of chunks ``0..r``.  They are brought in
with one all-gather along the sequence (keys and values are ``Hkv / Hq`` of the query volume under
GQA, so this moves far less than gathering activations would); the rank then runs the flash
attention kernel on ``q_local [B, S/W]`` against the prefix ``K, V [B, (r+1) S/W]`` with the causal
diagonal aligned bottom-right, which the kernel supports directly.  Backward runs the attention
backward kernel on the same operands and returns the key / value gradients to their owners with a
reduce-scatter along the sequence.

The reference exposes ``context_parallel_size`` (Megatron) and ``sp_size`` (FLUX, Ulysses-style) as
knobs that are 1 in every shipped configuration
(llama2_sft/primus/conf/llama2_70b_lora_posttrain.yaml:22; flux1/primus/conf/flux.1_schnell_t2i-pretrain.yaml:48;
llama2_sft/primus/src/llama2_custom.py:393-397).  The work per rank grows with ``r`` (a zig-zag
chunk assignment would balance it); correctness does not depend on the assignment.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
from torch.autograd import Function

from ..ops import kernels as K


def _all_gather_seq(t: torch.Tensor, group, world: int) -> torch.Tensor:
    """``[B, s, H, D]`` -> ``[B, world * s, H, D]``."""
    parts = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(parts, t.contiguous(), group=group)
    return torch.cat(parts, dim=1)


def _reduce_scatter_seq(t: torch.Tensor, group, world: int, rank: int) -> torch.Tensor:
    """``[B, world * s, H, D]`` summed over ranks -> this rank's ``[B, s, H, D]``."""
    t = t.contiguous()
    if t.is_cuda:
        chunks = [c.contiguous() for c in t.chunk(world, dim=1)]
        out = torch.empty_like(chunks[0])
        dist.reduce_scatter(out, chunks, group=group)
        return out
    dist.all_reduce(t, group=group)
    return t.chunk(world, dim=1)[rank].contiguous()


class ContextParallelAttentionFn(Function):
    @staticmethod
    def forward(ctx, q, k, v, group, scale, window):
        W, r = dist.get_world_size(group), dist.get_rank(group)
        s = q.shape[1]
        kf = _all_gather_seq(k, group, W)[:, :(r + 1) * s].contiguous()
        vf = _all_gather_seq(v, group, W)[:, :(r + 1) * s].contiguous()
        q = q.contiguous()
        out, lse = K.attention_fwd(q, kf, vf, scale=scale, causal=True, window=window)
        ctx.save_for_backward(q, kf, vf, out, lse)
        ctx.cfg = (group, W, r, scale, window, k.dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, kf, vf, out, lse = ctx.saved_tensors
        group, W, r, scale, window, kdt = ctx.cfg
        dq, dk, dv, _ = K.attention_bwd(dout.contiguous(), q, kf, vf, out, lse, scale=scale, causal=True, window=window)
        s = q.shape[1]
        full = (q.shape[0], W * s, kf.shape[2], kf.shape[3])
        dk_full = torch.zeros(full, dtype=torch.float32, device=q.device)
        dv_full = torch.zeros(full, dtype=torch.float32, device=q.device)
        dk_full[:, :(r + 1) * s] = dk.float()
        dv_full[:, :(r + 1) * s] = dv.float()
        dk_l = _reduce_scatter_seq(dk_full, group, W, r)
        dv_l = _reduce_scatter_seq(dv_full, group, W, r)
        return dq.to(q.dtype), dk_l.to(kdt), dv_l.to(kdt), None, None, None


def context_parallel_attention(q, k, v, group, *, scale: float | None = None, window: int = 0) -> torch.Tensor:
    """Causal attention over a sequence sharded across ``group``; ``q [B, S/W, Hq, D]``,
    ``k``/``v`` ``[B, S/W, Hkv, D]`` are this rank's chunk (chunk index = rank in the group)."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    if group is None or dist.get_world_size(group) == 1:
        from ..ops.functional import attention
        return attention(q, k, v, causal=True, window=window, scale=scale)
    return ContextParallelAttentionFn.apply(q, k, v, group, scale, window)
