"""Expert parallelism: token dispatch / combine over an expert-parallel group.

``ExpertParallelDispatcher`` is the collective-library path (``all_to_all_single`` with split
sizes exchanged first), the analogue of Megatron's ``alltoall`` token dispatcher that the reference
selects (gpt_oss_20B-MXFP4-deosc-mlperf-pretrain.yaml:164) and the baseline the fused peer-memory
dispatch is measured against.  Flow per layer:

    source rank : sort (token, slot) pairs by global expert -> rows grouped by destination rank
    all-to-all  : per-(rank, expert) counts, then the rows themselves
    owner rank  : regroup received rows by local expert (128-row padded segments), grouped MLP,
                  undo the regrouping
    all-to-all  : rows back to their source rank
    source rank : weighted sum over the k slots of every token

Every step is an autograd Function whose backward is the mirrored step, so the same code serves
forward and backward.  Works on NCCL and on gloo (CPU tests).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch.autograd import Function

from ..ops import moe_ops as M


class _AllToAllRows(Function):
    @staticmethod
    def forward(ctx, x, in_splits, out_splits, group):
        ctx.cfg = (in_splits, out_splits, group)
        out = torch.empty((sum(out_splits), x.shape[1]), dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        in_splits, out_splits, group = ctx.cfg
        out = torch.empty((sum(in_splits), g.shape[1]), dtype=g.dtype, device=g.device)
        dist.all_to_all_single(out, g.contiguous(), in_splits, out_splits, group=group)
        return out, None, None, None


class ExpertParallelDispatcher:
    def __init__(self, group, n_experts: int):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.E = n_experts
        self.local = n_experts // self.world

    def __call__(self, x, idx, w, counts, w1, w2):
        T, k = idx.shape
        W, L = self.world, self.local
        # 1. rows sorted by global expert, unpadded (pad = 1): destination ranks are contiguous
        seg, _, dest, _ = M.plan(idx, counts, self.E, pad=1)
        rows = T * k
        send = M.PermuteFn.apply(x, dest, k, rows)
        # 2. counts exchange: recv_counts[s, l] = pairs rank s sends to my local expert l
        send_counts = counts.view(W, L).to(torch.int64)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts.contiguous(), group=self.group)
        in_splits = send_counts.sum(1).tolist()        # host read: the collective needs sizes
        out_splits = recv_counts.sum(1).tolist()
        recv = _AllToAllRows.apply(send, in_splits, out_splits, self.group)
        # 3. regroup by local expert: received rows are ordered (source rank, local expert)
        n_recv = recv.shape[0]
        local_idx = torch.repeat_interleave(torch.arange(L, device=x.device).repeat(W), recv_counts.reshape(-1),
                                            output_size=n_recv).to(torch.int32).view(-1, 1)
        local_counts = recv_counts.sum(0).to(torch.int32)
        seg2, tile_expert, dest2, rows2 = M.plan(local_idx, local_counts, L)
        xp = M.PermuteFn.apply(recv, dest2, 1, rows2)
        yp = M.GroupedMLPFn.apply(xp, w1, w2, seg2, tile_expert)
        back = M.UnpermuteFn.apply(yp, dest2, None, n_recv, 1)
        # 4. return trip and weighted combine at the source
        ret = _AllToAllRows.apply(back, out_splits, in_splits, self.group)
        return M.UnpermuteFn.apply(ret, dest, w, T, k)
