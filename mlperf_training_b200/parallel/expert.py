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

    def __call__(self, x, idx, w, counts, w1, w2, precision: str = "bf16"):
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
        seg2, tile_expert, dest2, rows2 = M.plan(local_idx, local_counts, L, pad=M.pad_rows(precision))
        xp = M.PermuteFn.apply(recv, dest2, 1, rows2)
        yp = M.grouped_mlp(xp, w1, w2, seg2, tile_expert, precision)
        back = M.UnpermuteFn.apply(yp, dest2, None, n_recv, 1)
        # 4. return trip and weighted combine at the source
        ret = _AllToAllRows.apply(back, out_splits, in_splits, self.group)
        return M.UnpermuteFn.apply(ret, dest, w, T, k)


# --------------------------------------------------------------------------------------
# peer-memory path
# --------------------------------------------------------------------------------------
class _Route:
    """Per-layer routing tables, all on the device (no size is read back to the host)."""
    __slots__ = ("dst_rank", "dst_row", "seg2", "cnt2", "tile_expert", "n")


class _PushRows(Function):
    """rows [n, D] (this rank's pairs in sorted order) -> the owners' slabs; returns this rank's slab
    (rows of every source, grouped by local expert, padding zero).  Backward pulls the gradient rows
    of this rank's pairs out of the owners' gradient slabs."""

    @staticmethod
    def forward(ctx, rows, disp, route: _Route):
        ctx.disp, ctx.route = disp, route
        return disp._push(rows, route, disp.slab_x)

    @staticmethod
    def backward(ctx, g_slab):
        return ctx.disp._pull(g_slab, ctx.route, ctx.disp.slab_dx), None, None


class _PullRows(Function):
    """slab [cap, D] (expert outputs on the owner) -> rows [n, D] of this rank's pairs, loaded from
    the owners' slabs.  Backward pushes the gradient rows into the owners' gradient slabs."""

    @staticmethod
    def forward(ctx, slab, disp, route: _Route):
        ctx.disp, ctx.route = disp, route
        return disp._pull(slab, route, disp.slab_y)

    @staticmethod
    def backward(ctx, g_rows):
        return ctx.disp._push(g_rows.contiguous(), ctx.route, ctx.disp.slab_dy), None, None


class FusedExpertDispatcher:
    """Token dispatch / combine by this package's kernels over NVLink peer memory.

    Every rank owns four symmetric slabs ``[capacity, D]`` (inputs, outputs and their gradients).
    Dispatch stores each (token, slot) row directly at its final, expert-grouped position in the
    owner's slab; combine loads each pair's output row from the owner's slab.  Positions come from
    the all-gathered per-expert counts by prefix sums on the device, so the layer runs without a
    host synchronisation; ``capacity`` bounds the rows a rank can receive (``capacity_factor`` x the
    balanced share) and pairs beyond it are dropped and counted in ``dropped``.
    """

    def __init__(self, group, n_experts: int, hidden: int, max_pairs: int, device, capacity_factor: float = 2.0,
                 share_with: "FusedExpertDispatcher | None" = None, pad: int = M.PAD):
        from .symm import SymmetricBuffer
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.E, self.D = n_experts, hidden
        self.local = n_experts // self.world
        self.pad = pad                     # row padding of an expert segment (the grouped kernels' row tile)
        self.cap = (int(capacity_factor * max_pairs) + self.local * pad + pad - 1) // pad * pad
        mk = lambda: SymmetricBuffer(self.cap * hidden, torch.bfloat16, group, device)
        # The input slab is read again in backward (weight gradients), so every layer owns one; the
        # output and gradient slabs are consumed right after they are filled and are shared between the
        # layers that pass ``share_with``.
        self.slab_x = mk()
        if share_with is not None and share_with.cap == self.cap and share_with.D == hidden:
            self.slab_y, self.slab_dy, self.slab_dx = share_with.slab_y, share_with.slab_dy, share_with.slab_dx
            self.dropped = share_with.dropped
        else:
            self.slab_y, self.slab_dy, self.slab_dx = mk(), mk(), mk()
            self.dropped = torch.zeros(1, dtype=torch.int32, device=device)
        self.device = device

    # ------------------------------------------------------------------ routing tables
    def _route(self, counts: torch.Tensor, seg: torch.Tensor, n: int) -> _Route:
        W, L, E, dev = self.world, self.local, self.E, counts.device
        from ..ops import _lib
        if _lib.use_kernels(counts):
            # one exchange of the per-expert counts, then every table in one kernel
            allc32 = torch.empty((W, E), dtype=torch.int32, device=dev)
            dist.all_gather_into_tensor(allc32.view(-1), counts.to(torch.int32).contiguous(), group=self.group)
            r = _Route()
            r.n = n
            r.dst_rank = torch.empty(n, dtype=torch.int32, device=dev)
            r.dst_row = torch.empty(n, dtype=torch.int32, device=dev)
            r.seg2 = torch.empty(L + 1, dtype=torch.int32, device=dev)
            r.cnt2 = torch.empty(L, dtype=torch.int32, device=dev)
            r.tile_expert = torch.empty(self.cap // self.pad, dtype=torch.int32, device=dev)
            _lib.call("b200_ep_route", _lib.ptr(allc32), _lib.ptr(seg.to(torch.int32).contiguous()), W, E, self.rank, self.pad,
                      self.cap, n, _lib.ptr(r.dst_rank), _lib.ptr(r.dst_row), _lib.ptr(r.seg2), _lib.ptr(r.cnt2),
                      _lib.ptr(r.tile_expert), _lib.stream_ptr())
            return r
        allc = torch.empty((W, E), dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(allc.view(-1), counts.to(torch.int64).contiguous(), group=self.group)
        tot = allc.sum(0)                                            # rows every expert receives
        pad = self.pad
        padded = (tot + pad - 1) // pad * pad
        seg_all = (padded.view(W, L).cumsum(1) - padded.view(W, L)).reshape(-1)      # segment start on the owner
        before_me = allc[: self.rank].sum(0)                         # rows of lower ranks inside the segment
        base = seg_all + before_me
        e_of = torch.repeat_interleave(torch.arange(E, device=dev), counts.long(), output_size=n)
        r = _Route()
        r.n = n
        r.dst_rank = (e_of // L).to(torch.int32)
        row = base[e_of] + (torch.arange(n, device=dev) - seg.long()[e_of])
        r.dst_row = torch.where(row < self.cap, row, torch.full_like(row, -1)).to(torch.int32)
        mine = slice(self.rank * L, (self.rank + 1) * L)
        seg2 = torch.zeros(L + 1, dtype=torch.int64, device=dev)
        seg2[1:] = padded[mine].cumsum(0)
        r.seg2 = seg2.clamp(max=self.cap).to(torch.int32)
        r.cnt2 = tot[mine].to(torch.int32)
        tile_start = torch.arange(self.cap // pad, device=dev) * pad
        te = torch.searchsorted(seg2[1:].contiguous(), tile_start, right=True)
        r.tile_expert = torch.where(tile_start < seg2[-1], te, torch.full_like(te, -1)).to(torch.int32)
        return r

    # ------------------------------------------------------------------ data movement
    def _push(self, rows: torch.Tensor, route: _Route, slab) -> torch.Tensor:
        from ..ops import _lib
        slab.barrier()                         # every rank is done reading this slab from its previous use
        _lib.call("b200_zero_pad_rows", _lib.ptr(slab.local), _lib.ptr(route.seg2), _lib.ptr(route.cnt2), self.local, self.D,
                  self.cap, _lib.stream_ptr())
        _lib.call("b200_scatter_rows_to_peers", _lib.ptr(rows), None, _lib.ptr(route.dst_rank), _lib.ptr(route.dst_row),
                  route.n, self.D, slab.ptr_array(), self.world, self.cap, _lib.ptr(self.dropped), _lib.stream_ptr())
        slab.barrier()                         # every rank's rows have landed
        return slab.local.view(self.cap, self.D)

    def _pull(self, slab_rows: torch.Tensor, route: _Route, slab) -> torch.Tensor:
        from ..ops import _lib
        if slab_rows.data_ptr() != slab.local.data_ptr():
            slab.barrier()                     # previous readers of this slab are done
            slab.local.view(self.cap, self.D).copy_(slab_rows)
        # else: the expert GEMM wrote the slab in place.  Its previous readers (the peers' gathers of the layer
        # before) are ordered before that GEMM by the collective this layer ran since: the exchange of the counts in
        # forward, the barriers of the gradient push in backward.
        slab.barrier()                         # every owner's slab is complete
        out = torch.empty((route.n, self.D), dtype=torch.bfloat16, device=slab_rows.device)
        _lib.call("b200_gather_rows_from_peers", slab.ptr_array(), _lib.ptr(route.dst_rank), _lib.ptr(route.dst_row),
                  route.n, self.D, _lib.ptr(out), self.world, self.cap, _lib.stream_ptr())
        return out

    def __call__(self, x, idx, w, counts, w1, w2, precision: str = "bf16"):
        T, k = idx.shape
        n = T * k
        seg, _, dest, _ = M.plan(idx, counts, self.E, pad=1)       # sorted by global expert, unpadded
        send = M.PermuteFn.apply(x, dest, k, n)
        route = self._route(counts, seg, n)
        xp = _PushRows.apply(send, self, route)
        yp = M.grouped_mlp(xp, w1, w2, route.seg2, route.tile_expert, precision,
                           y_out=self.slab_y.local.view(self.cap, self.D), dx_out=self.slab_dx.local.view(self.cap, self.D))
        ret = _PullRows.apply(yp, self, route)
        return M.UnpermuteFn.apply(ret, dest, w, T, k)
