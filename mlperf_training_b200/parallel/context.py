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


# --------------------------------------------------------------------------------------
# Ulysses-style sequence parallelism: exchange sequence shards for head shards around attention
# --------------------------------------------------------------------------------------
class _SeqToHeads(Function):
    """``[B, S/W, H, D]`` (all heads, this rank's sequence chunk) -> ``[B, S, H/W, D]`` (whole
    sequence, this rank's heads) with one all-to-all; backward is the inverse exchange."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _a2a_seq_heads(x, group, to_heads=True)

    @staticmethod
    def backward(ctx, g):
        return _a2a_seq_heads(g.contiguous(), ctx.group, to_heads=False), None


class _HeadsToSeq(Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _a2a_seq_heads(x, group, to_heads=False)

    @staticmethod
    def backward(ctx, g):
        return _a2a_seq_heads(g.contiguous(), ctx.group, to_heads=True), None


def _a2a_seq_heads(x: torch.Tensor, group, to_heads: bool) -> torch.Tensor:
    W = dist.get_world_size(group)
    B, s, H, D = x.shape
    if to_heads:
        if H % W:
            raise ValueError(f"{H} heads do not divide over {W} ranks")
        # piece j (heads of rank j) of my sequence chunk goes to rank j; I receive chunk i of my heads from rank i
        send = x.view(B, s, W, H // W, D).permute(2, 0, 1, 3, 4).contiguous()          # [W, B, s, H/W, D]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)
        return recv.permute(1, 0, 2, 3, 4).reshape(B, W * s, H // W, D)                  # chunks in rank order = sequence order
    S = s                                                                                 # here x is [B, S, H/W, D]
    send = x.view(B, W, S // W, H, D).permute(1, 0, 2, 3, 4).contiguous()                # [W, B, S/W, h, D]: chunk i -> rank i
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv.permute(1, 2, 0, 3, 4).reshape(B, S // W, W * H, D)                      # heads of rank j in slot j


def ulysses_attention(q, k, v, group, *, causal: bool = False, window: int = 0, scale: float | None = None) -> torch.Tensor:
    """Attention over a sequence sharded across ``group`` by exchanging the sharded dimension: two
    all-to-alls turn (all heads, S/W tokens) into (H/W heads, all tokens), the local flash-attention
    kernel runs on whole sequences, and one all-to-all brings the output back.  Needs the number of
    query and of key/value heads to be divisible by the group size (the ``sp_size`` knob of the
    reference's diffusion trainer, flux1/primus/conf/flux.1_schnell_t2i-pretrain.yaml:48)."""
    from ..ops.functional import attention
    if group is None or dist.get_world_size(group) == 1:
        return attention(q, k, v, causal=causal, window=window, scale=scale)
    qh, kh, vh = (_SeqToHeads.apply(t.contiguous(), group) for t in (q, k, v))
    oh = attention(qh, kh, vh, causal=causal, window=window, scale=scale)
    return _HeadsToSeq.apply(oh.contiguous(), group)
