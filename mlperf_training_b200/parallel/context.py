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
llama2_sft/primus/src/llama2_custom.py:393-397).  In this all-gather form the work per rank grows with ``r``.

``ring_attention`` is the balanced form (Megatron's default ``cp_comm_type`` p2p, which the reference's provider gets with
``context_parallel_size > 1``: llama2_sft/primus/src/llama2_custom.py:393-397,501-506): the sequence is cut into
``2 W`` chunks and rank ``r`` holds chunks ``r`` and ``2 W - 1 - r`` (zig-zag), key / value blocks travel round
the ring with point-to-point messages posted before the attention of the block in hand, the partial outputs
are merged by their log-sum-exp, and every ring step costs every rank the same half block of work.  Memory
stays at one visiting key / value block instead of the whole prefix.
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
# Ring attention over zig-zag chunks
# --------------------------------------------------------------------------------------
def zigzag_chunk(t: torch.Tensor, world: int, rank: int, dim: int = 1) -> torch.Tensor:
    """Chunks ``rank`` and ``2 * world - 1 - rank`` of the ``2 * world`` equal chunks of ``t`` along ``dim``."""
    if t.shape[dim] % (2 * world):
        raise ValueError(f"length {t.shape[dim]} does not divide into {2 * world} zig-zag chunks")
    parts = t.chunk(2 * world, dim=dim)
    return torch.cat([parts[rank], parts[2 * world - 1 - rank]], dim=dim).contiguous()


def zigzag_unchunk(parts: list, dim: int = 1) -> torch.Tensor:
    """Inverse of ``zigzag_chunk`` over the list of every rank's piece."""
    W = len(parts)
    halves = [p.chunk(2, dim=dim) for p in parts]
    return torch.cat([halves[r][0] for r in range(W)] + [halves[W - 1 - r][1] for r in range(W)], dim=dim)


def _block_bwd(dout, q, k, v, out, lse, scale, causal):
    """Gradients of one (query block, key / value block) pair of an attention whose softmax is normalised by the
    GLOBAL ``lse`` (and whose ``out`` is the merged output): ``P = exp(S - lse)``, ``dS = P (dP - rowsum(dO O))``.
    Returns fp32 ``(dq, dk, dv)``."""
    if q.is_cuda:
        dq, dk, dv, _ = K.attention_bwd(dout.contiguous(), q.contiguous(), k.contiguous(), v.contiguous(), out.contiguous(),
                                        lse.contiguous(), scale=scale, causal=causal)
        return dq.float(), dk.float(), dv.float()
    B, Sq, Hq, D = q.shape
    Skv, Hkv = k.shape[1], k.shape[2]
    g = Hq // Hkv
    qf, do, of = q.float(), dout.float(), out.float()
    kf, vf = k.float().repeat_interleave(g, dim=2), v.float().repeat_interleave(g, dim=2)
    sc = torch.einsum("bqhd,bkhd->bhqk", qf, kf) * scale
    if causal:
        vis = torch.arange(Skv)[None, :] <= torch.arange(Sq)[:, None] + (Skv - Sq)
        sc = sc.masked_fill(~vis, float("-inf"))
    p = torch.exp(sc - lse[..., None])
    delta = (do * of).sum(-1).transpose(1, 2)                                   # [B, Hq, Sq]
    dv = torch.einsum("bhqk,bqhd->bkhd", p, do)
    dp = torch.einsum("bqhd,bkhd->bhqk", do, vf)
    ds = p * (dp - delta[..., None])
    dq = torch.einsum("bhqk,bkhd->bqhd", ds, kf) * scale
    dk = torch.einsum("bhqk,bqhd->bkhd", ds, qf) * scale
    return dq, dk.view(B, Skv, Hkv, g, D).sum(3), dv.view(B, Skv, Hkv, g, D).sum(3)


def _ring_exchange(send: list, recv_like: list, nxt: int, prv: int, group):
    """Post the sends to the next rank and the receives from the previous one together; returns (requests, buffers)."""
    ops, bufs = [], []
    for t in send:
        ops.append(dist.P2POp(dist.isend, t, nxt, group))
    for t in recv_like:
        b = torch.empty_like(t)
        bufs.append(b)
        ops.append(dist.P2POp(dist.irecv, b, prv, group))
    return (dist.batch_isend_irecv(ops) if ops else []), bufs


class RingAttentionFn(Function):
    """Causal attention with ``q``, ``k``, ``v`` ``[B, 2 c, H, D]`` holding this rank's two zig-zag chunks.  At ring
    step ``t`` the rank holds the keys / values of rank ``j = (r - t) mod W``: its own (``t = 0``: causal attention
    over the local rows - the first chunk precedes the second), an earlier rank's (``j < r``: every query sees the
    visitor's first chunk, nothing of its second) or a later rank's (``j > r``: only the queries of the second chunk
    see the visitor, all of it)."""

    @staticmethod
    def forward(ctx, q, k, v, group, scale):
        W, r = dist.get_world_size(group), dist.get_rank(group)
        ranks = dist.get_process_group_ranks(group)
        nxt, prv = ranks[(r + 1) % W], ranks[(r - 1) % W]
        c = q.shape[1] // 2
        q = q.contiguous()
        kv = torch.stack([k, v]).contiguous()
        out = lse = None
        for t in range(W):
            reqs, bufs = _ring_exchange([kv], [kv], nxt, prv, group) if t + 1 < W else ([], [])
            j = (r - t) % W
            if t == 0:
                o, l = K.attention_fwd(q, kv[0], kv[1], scale=scale, causal=True)
                out, lse = o.float(), l.clone()
            else:
                lo = 0 if j < r else c                                          # the query rows that see the visitor
                kk, vv = (kv[0][:, :c], kv[1][:, :c]) if j < r else (kv[0], kv[1])
                o, l = K.attention_fwd(q[:, lo:].contiguous(), kk.contiguous(), vv.contiguous(), scale=scale, causal=False)
                new = torch.logaddexp(lse[:, :, lo:], l)
                w_old = torch.exp(lse[:, :, lo:] - new).transpose(1, 2)[..., None]
                w_new = torch.exp(l - new).transpose(1, 2)[..., None]
                out[:, lo:] = out[:, lo:] * w_old + o.float() * w_new
                lse[:, :, lo:] = new
            for w in reqs:
                w.wait()
            if bufs:
                kv = bufs[0]
        out = out.to(q.dtype)
        ctx.save_for_backward(q, k.contiguous(), v.contiguous(), out, lse)
        ctx.cfg = (group, W, r, nxt, prv, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        group, W, r, nxt, prv, scale = ctx.cfg
        c = q.shape[1] // 2
        dout = dout.contiguous()
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        kv = torch.stack([k, v]).contiguous()
        dkv = torch.zeros(kv.shape, dtype=torch.float32, device=q.device)     # travels with the block it belongs to
        for t in range(W):
            reqs, bufs = _ring_exchange([kv], [kv], nxt, prv, group) if t + 1 < W else ([], [])
            j = (r - t) % W
            if t == 0:
                a, b, d = _block_bwd(dout, q, kv[0], kv[1], out, lse, scale, True)
                dq += a
                dkv[0] += b
                dkv[1] += d
            elif j < r:
                a, b, d = _block_bwd(dout, q, kv[0][:, :c], kv[1][:, :c], out, lse, scale, False)
                dq += a
                dkv[0][:, :c] += b
                dkv[1][:, :c] += d
            else:
                a, b, d = _block_bwd(dout[:, c:], q[:, c:], kv[0], kv[1], out[:, c:], lse[:, :, c:], scale, False)
                dq[:, c:] += a
                dkv[0] += b
                dkv[1] += d
            for w in reqs:
                w.wait()
            # the gradient block follows its keys / values; after the last step it arrives at its owner
            greqs, gbufs = _ring_exchange([dkv], [dkv], nxt, prv, group)
            for w in greqs:
                w.wait()
            dkv = gbufs[0]
            if bufs:
                kv = bufs[0]
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, None


def ring_attention(q, k, v, group, *, scale: float | None = None) -> torch.Tensor:
    """Causal attention over a sequence sharded across ``group`` in zig-zag order: ``q [B, S / W, Hq, D]`` and
    ``k`` / ``v`` hold chunks ``r`` and ``2 W - 1 - r`` of the ``2 W`` chunks of the sequence (``zigzag_chunk``)."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    if group is None or dist.get_world_size(group) == 1:
        from ..ops.functional import attention
        return attention(q, k, v, causal=True, scale=scale)
    if q.shape[1] % 2:
        raise ValueError("ring attention needs an even number of rows per rank (two zig-zag chunks)")
    return RingAttentionFn.apply(q, k, v, group, scale)


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
