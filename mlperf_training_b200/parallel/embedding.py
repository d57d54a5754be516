"""Row-wise sharded embedding table with a sparse optimizer applied in backward.

Rank ``r`` of ``W`` owns the contiguous rows ``[r * rows_per_rank, (r + 1) * rows_per_rank)`` of the
table (TorchRec's ROW_WISE sharding; the state dict exposes the shard with its global row offset
under ``embeddings.<table>.weight`` so a TorchRec-style loader can place it).  A lookup is

    dedup ids -> bucketise by owner -> exchange request counts and ids ->
    owners read their rows -> rows travel back to the requesters -> expand to the original order

and backward mirrors it: duplicate gradient rows are summed in sorted (fixed) order by a segment
reduction over the forward's sort permutation, sent to the owners in the wire dtype (bf16 for a bf16
table: the quantised gradient exchange of generative_recommenders/dlrm_v4/train/utils.py:1136-1308),
sorted and summed again per unique row there and applied with row-wise Adagrad immediately
(``apply_optimizer_in_backward`` in the reference, generative_recommenders/dlrm_v4/train/utils.py:1547-1783).
Dedup, sort, run offsets and both reductions are device kernels (``ops.sort``: bounded-key radix sort,
no atomics); the one host read per lookup is the vector of per-owner request counts that sizes the
exchange.

``comm="nccl"`` moves the rows with ``all_to_all_single`` (the TorchRec / RCCL structure of the
reference and the baseline here).  ``comm="fused"`` is the in-kernel NVLink path: the owner's
gather kernel stores every requested row straight into the requester's symmetric receive buffer
(``gather_rows_to_peers``), so the row all-to-all and the lookup are one kernel.  With a single
rank both reduce to a local gather.
"""
from __future__ import annotations

import ctypes
import itertools

import torch
import torch.distributed as dist
from torch.autograd import Function

from ..ops import _lib
from ..ops import kernels as K
from ..ops import sort as S


class ShardedEmbedding:
    def __init__(self, rows: int, dim: int, *, group=None, device="cpu", dtype=torch.bfloat16, lr: float = 1e-2,
                 eps: float = 1e-8, seed: int = 0, init_scale: float | None = None, comm: str = "nccl",
                 max_requests: int = 1 << 20, name: str = "item", owner: int | None = None):
        self.group = group
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.rows, self.dim, self.name = rows, dim, name
        self.device = torch.device(device)
        # row ranges per rank: ROW_WISE cuts the table evenly; TABLE_WISE (``owner`` given) puts every row on one rank.
        # Either way rank r owns rows [bounds[r], bounds[r + 1]) and the same routing serves both.
        self.owner = owner
        if owner is None:
            self.rows_per_rank = (rows + self.world - 1) // self.world
            bounds = [min(r * self.rows_per_rank, rows) for r in range(self.world + 1)]
        else:
            self.rows_per_rank = rows
            bounds = [0 if r <= owner else rows for r in range(self.world + 1)]
        self.bounds = torch.tensor(bounds, dtype=torch.int64, device=self.device)
        self.row_lo = bounds[self.rank]
        self.local_rows = bounds[self.rank + 1] - bounds[self.rank]
        g = torch.Generator(device=self.device).manual_seed(seed * 7919 + self.rank)
        scale = init_scale if init_scale is not None else (1.0 / rows) ** 0.5
        self.weight = (torch.rand(self.local_rows, dim, generator=g, device=self.device) * 2 - 1).mul_(scale).to(dtype)
        self.state = torch.zeros(self.local_rows, dtype=torch.float32, device=self.device)   # Adagrad row sums
        self.lr, self.eps = lr, eps
        self.comm = comm if (self.world > 1 and self.device.type == "cuda") else "nccl"
        self.recv = None
        import os
        self._verify_left = int(os.environ.get("B200_VERIFY_FUSED_LOOKUP", "0") or 0)     # compare the first N fused lookups
        if self.comm == "fused":
            from .symm import SymmetricBuffer
            self.max_requests = max_requests
            self.recv = SymmetricBuffer(max_requests * dim, dtype, group, self.device)

    # ------------------------------------------------------------------ routing
    def _route(self, ids: torch.Tensor):
        """Dedup + bucketise.  Returns ``(uniq_sorted_by_owner, inverse, send_counts [W], sorted)``."""
        srt = S.sort_unique(ids, S.key_bits_for(self.rows))                      # sorted ids = sorted by owner
        n = ids.numel()
        valid = torch.arange(n, device=ids.device) < srt.count
        own = torch.bucketize(srt.uniq, self.bounds[1:], right=True).clamp(max=self.world - 1)
        owner = torch.where(valid, own, self.world)
        counts = torch.bincount(owner, minlength=self.world + 1)[: self.world]
        head = torch.cat([srt.count.reshape(1), counts]).tolist()                # the lookup's one host read
        self._last_counts = head[1:]
        return srt.uniq[: head[0]], srt.inverse, counts, srt

    def _exchange_ids(self, uniq, send_counts):
        W = self.world
        if W == 1:
            return uniq - self.row_lo, self._last_counts, self._last_counts, None
        counts = torch.empty((W, W), dtype=torch.int64, device=uniq.device)
        dist.all_gather_into_tensor(counts.view(-1), send_counts.to(torch.int64), group=self.group) \
            if uniq.is_cuda else dist.all_gather(list(counts.unbind(0)), send_counts.to(torch.int64), group=self.group)
        counts_h = counts.tolist()                                  # counts_h[s][o]: rank s asks owner o
        in_splits = counts_h[self.rank]
        out_splits = [counts_h[s][self.rank] for s in range(W)]
        recv_ids = torch.empty(sum(out_splits), dtype=torch.int64, device=uniq.device)
        dist.all_to_all_single(recv_ids, uniq.contiguous(), out_splits, in_splits, group=self.group)
        return recv_ids - self.row_lo, in_splits, out_splits, counts_h

    # ------------------------------------------------------------------ forward / backward
    def input_dist(self, ids: torch.Tensor) -> dict:
        """The id half of a lookup: sort / dedup, bucketise by owner, exchange request counts and ids.
        It depends on the batch's ids only, so a pipelined trainer runs it for batch N + 1 on a side
        stream while batch N computes, and hands the plan to ``lookup`` later (the sparse-data-dist stage
        of the reference's ``_StreamingTrainPipeline``, generative_recommenders/dlrm_v4/train/utils.py:3487-3871)."""
        uniq, inverse, send_counts, srt = self._route(ids.reshape(-1))
        local_idx, in_splits, out_splits, counts_h = self._exchange_ids(uniq, send_counts)
        return {"uniq": uniq, "inverse": inverse, "srt": srt, "local_idx": local_idx, "in_splits": in_splits,
                "out_splits": out_splits, "counts_h": counts_h}

    def lookup(self, ids: torch.Tensor, plan: dict | None = None) -> torch.Tensor:
        """``ids`` int64 ``[n]`` (global row ids) -> rows ``[n, dim]``; differentiable.  ``plan``: the result
        of an earlier ``input_dist(ids)`` for the same ids."""
        return _LookupFn.apply(ids, self, torch.empty(0, requires_grad=True, device=ids.device), plan)

    def _forward_rows(self, ids, plan: dict | None = None):
        plan = plan if plan is not None else self.input_dist(ids)
        uniq, inverse, srt = plan["uniq"], plan["inverse"], plan["srt"]
        local_idx, in_splits, out_splits, counts_h = plan["local_idx"], plan["in_splits"], plan["out_splits"], plan["counts_h"]
        W = self.world
        if W == 1:
            rows_u = K.gather_rows(self.weight, local_idx)
        elif self.comm == "fused":
            n_u = uniq.numel()
            if n_u > self.max_requests:
                raise RuntimeError(f"{n_u} unique ids exceed the receive buffer ({self.max_requests})")
            recv_off = torch.tensor([0] + list(itertools.accumulate(out_splits)), dtype=torch.int64, device=ids.device)
            # where my segment starts inside requester s's buffer: its requests to owners before me
            base_rows = (ctypes.c_longlong * W)(*[sum(counts_h[s][:self.rank]) for s in range(W)])
            self.recv.barrier()                                   # previous consumers are done with the buffers
            _lib.call("b200_gather_rows_to_peers", _lib.ptr(self.weight), self.local_rows, _lib.ptr(local_idx),
                      _lib.ptr(recv_off), int(sum(out_splits)), W, self.dim, self.recv.ptr_array(), base_rows,
                      _lib.stream_ptr())
            self.recv.barrier()                                   # every owner's rows have landed
            rows_u = self.recv.local[: n_u * self.dim].view(n_u, self.dim).clone()
            if self._verify_left > 0:
                # first calls of a run, on request: the same rows through the library all-to-all, compared bit for bit
                # (the reference arms its fused exchanges the same way: DLRM_HSTU_FP8_SEQ_A2A_FUSED_VERIFY,
                # generative_recommenders/dlrm_v4/seq_a2a_rowperm.py:752-772)
                self._verify_left -= 1
                served = K.gather_rows(self.weight, local_idx)
                ref = torch.empty_like(rows_u)
                dist.all_to_all_single(ref, served, in_splits, out_splits, group=self.group)
                if not torch.equal(ref, rows_u):
                    raise RuntimeError(f"table {self.name}: the peer-store lookup differs from the all-to-all lookup "
                                       f"({int((ref != rows_u).any(1).sum())} of {n_u} rows)")
        else:
            served = K.gather_rows(self.weight, local_idx)
            rows_u = torch.empty((uniq.numel(), self.dim), dtype=self.weight.dtype, device=ids.device)
            dist.all_to_all_single(rows_u, served, in_splits, out_splits, group=self.group)
        return rows_u, (uniq, inverse, local_idx, in_splits, out_splits, srt)

    def _backward_rows(self, grad: torch.Tensor, ctx_state) -> None:
        uniq, inverse, local_idx, in_splits, out_splits, srt = ctx_state
        wire = torch.bfloat16 if self.weight.dtype == torch.bfloat16 else torch.float32
        if grad.dtype not in (torch.bfloat16, torch.float32):
            grad = grad.float()
        # 1. duplicates of this rank: one row per unique id, summed in sorted (fixed) order, in the wire dtype
        g_u = S.segment_sum(grad, srt, out_dtype=wire if self.world > 1 else torch.float32, max_seg=uniq.numel())
        # 2. to the owners
        if self.world > 1:
            recv = torch.empty((sum(out_splits), self.dim), dtype=wire, device=grad.device)
            dist.all_to_all_single(recv, g_u, out_splits, in_splits, group=self.group)
            g_u = recv
            # 3. several ranks may have asked for the same row: sort the requests, reduce per local row (fp32)
            srt_l = S.sort_unique(local_idx, S.key_bits_for(max(self.local_rows, 2)))
            g_l = S.segment_sum(g_u, srt_l, out_dtype=torch.float32)
            rows_l = srt_l.uniq                        # entries past the run count are -1: the update skips them
        else:
            g_l, rows_l = g_u, local_idx               # already one row per unique id
        self.apply_rowwise_adagrad(rows_l, g_l)

    def apply_rowwise_adagrad(self, rows: torch.Tensor, grads: torch.Tensor) -> None:
        """Row-wise Adagrad on the rows ``rows`` of the local shard (entries outside ``[0, local_rows)`` are skipped);
        the row width is the shard's own (a column-wise shard holds a slice of the table's width)."""
        if rows.numel() == 0:
            return
        if self.weight.is_cuda and self.weight.dtype == torch.bfloat16:
            _lib.call("b200_rowwise_adagrad", _lib.ptr(self.weight), _lib.ptr(self.state), _lib.ptr(rows.contiguous()),
                      _lib.ptr(grads.contiguous()), rows.numel(), self.weight.shape[1], float(self.lr), float(self.eps),
                      self.local_rows, _lib.stream_ptr())
            return
        ok = (rows >= 0) & (rows < self.local_rows)
        rows, grads = rows[ok], grads[ok]
        st = self.state[rows] + (grads * grads).mean(-1)
        self.state[rows] = st
        upd = self.weight[rows].float() - self.lr * grads / (st.sqrt()[:, None] + self.eps)
        self.weight[rows] = upd.to(self.weight.dtype)

    # ------------------------------------------------------------------ state dict (TorchRec-style shard metadata)
    def state_dict(self) -> dict:
        key = f"embeddings.{self.name}.weight"
        return {key: self.weight, f"{key}.row_offset": self.row_lo, f"{key}.global_rows": self.rows,
                f"embeddings.{self.name}.rowwise_adagrad.sum": self.state}

    def load_state_dict(self, sd: dict) -> None:
        key = f"embeddings.{self.name}.weight"
        if int(sd[f"{key}.row_offset"]) != self.row_lo or int(sd[f"{key}.global_rows"]) != self.rows:
            raise ValueError("embedding shard layout differs from the checkpoint (resharding is not supported here)")
        self.weight.copy_(sd[key])
        self.state.copy_(sd[f"embeddings.{self.name}.rowwise_adagrad.sum"])


    def snapshot(self):
        """Copies of the shard and its optimizer sums (warm-up steps are undone from them)."""
        return self.weight.clone(), self.state.clone()

    def restore(self, snap) -> None:
        self.weight.copy_(snap[0])
        self.state.copy_(snap[1])

    # ------------------------------------------------------------------ sharded (TorchRec-layout) state
    def sharded_state_dict(self, prefix: str = "") -> dict:
        """The table and its row-wise Adagrad sums as ``ShardedTensor``s over the table's group, under the key names a
        TorchRec ``EmbeddingCollection`` uses (``<prefix>embeddings.<table>.weight``; the fused optimizer state beside it):
        this rank's rows are one chunk at their row offset inside the ``[rows, dim]`` table, so a checkpoint written
        from it can be read back under another number of ranks or another placement (row-wise <-> table-wise).
        Collective over the group."""
        from torch.distributed._shard.sharded_tensor import Shard, ShardMetadata, init_from_local_shards
        if self.world == 1:
            return {f"{prefix}embeddings.{self.name}.weight": self.weight,
                    f"{prefix}embeddings.{self.name}.rowwise_adagrad.sum": self.state}
        owner = self.rank if (self.group is None or self.group is dist.group.WORLD) else dist.get_global_rank(self.group, self.rank)
        dev = f"rank:{owner}/{'cpu' if self.device.type == 'cpu' else str(self.device)}"
        out = {}
        for key, t, size in ((f"{prefix}embeddings.{self.name}.weight", self.weight, (self.rows, self.dim)),
                             (f"{prefix}embeddings.{self.name}.rowwise_adagrad.sum", self.state, (self.rows,))):
            shards = []
            if self.local_rows > 0:
                meta = ShardMetadata(shard_offsets=[int(self.row_lo)] + [0] * (t.dim() - 1), shard_sizes=list(t.shape), placement=dev)
                shards = [Shard(tensor=t, metadata=meta)]
            out[key] = init_from_local_shards(shards, *size, process_group=self.group)
        return out

    def save_sharded(self, path: str, prefix: str = "") -> None:
        """Write the sharded state with torch's distributed checkpoint writer (every rank its own rows)."""
        import torch.distributed.checkpoint as dcp
        dcp.save(self.sharded_state_dict(prefix), checkpoint_id=str(path))

    def load_sharded(self, path: str, prefix: str = "") -> None:
        """Read this rank's rows of a sharded checkpoint, whatever layout wrote it (the reader fetches the chunks that
        overlap this rank's row range)."""
        load_matching(self.sharded_state_dict(prefix), path)                    # the local shards are views of the live tensors


def load_matching(state: dict, path) -> list:
    """``dcp.load`` of the entries of ``state`` whose global shape equals the checkpoint's; returns the keys left
    out (the Adagrad sums of a column-wise table are ``[rows, shards]``: they do not carry over to or from a
    row-wise layout, and such a table then keeps the sums it has)."""
    import torch.distributed.checkpoint as dcp
    meta = dcp.FileSystemReader(str(path)).read_metadata().state_dict_metadata
    skipped = [k for k, v in state.items() if k in meta and hasattr(meta[k], "size")
               and tuple(meta[k].size) != tuple(v.size() if callable(getattr(v, "size", None)) else v.shape)]
    dcp.load({k: v for k, v in state.items() if k not in skipped}, checkpoint_id=str(path))
    return skipped


class _LookupFn(Function):
    @staticmethod
    def forward(ctx, ids, table: ShardedEmbedding, _anchor, plan=None):
        rows_u, st = table._forward_rows(ids.reshape(-1), plan)
        ctx.table, ctx.state = table, st
        return rows_u[st[1]]

    @staticmethod
    def backward(ctx, grad):
        ctx.table._backward_rows(grad.contiguous(), ctx.state)
        return None, None, None, None


class ColumnShardedEmbedding(ShardedEmbedding):
    """COLUMN_WISE sharding: rank ``r`` of ``W`` holds columns ``[r * dim / W, (r + 1) * dim / W)`` of EVERY row
    (TorchRec's placement for wide tables whose rows are hit unevenly: each rank serves the same number of
    rows per lookup whatever the id distribution, where ROW_WISE loads the owner of a hot row range).

    A lookup sends this rank's unique ids to every rank, each rank reads its column slice of all requested
    rows, and one all-to-all brings the ``W`` slices of a row back to its requester, which lays them side by
    side.  Backward cuts a gradient row into its ``W`` column slices, sends slice ``r`` to rank ``r``, reduces
    the requests of all ranks per row there (sorted order, fp32) and applies row-wise Adagrad to the slice.
    The Adagrad sum of a row is kept per column shard (the mean of squares runs over the shard's columns),
    which is how TorchRec's fused optimizer treats a column-wise shard: every shard is a table of its own.
    (The reference leaves the choice between row-, table- and column-wise placement to TorchRec's planner under its
    constraints: generative_recommenders/dlrm_v4/train/utils.py:1311-1545.)
    """

    def __init__(self, rows: int, dim: int, *, group=None, device="cpu", dtype=torch.bfloat16, lr: float = 1e-2,
                 eps: float = 1e-8, seed: int = 0, init_scale: float | None = None, name: str = "item", **_unused):
        self.group = group
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        if dim % self.world:
            raise ValueError(f"column-wise sharding needs the width ({dim}) to divide by the ranks ({self.world})")
        self.rows, self.dim, self.name = rows, dim, name
        self.device = torch.device(device)
        self.owner = None
        self.cols = dim // self.world
        self.col_lo = self.rank * self.cols
        self.rows_per_rank = self.local_rows = rows
        self.row_lo = 0
        self.bounds = torch.tensor([0] + [rows] * self.world, dtype=torch.int64, device=self.device)
        g = torch.Generator(device=self.device).manual_seed(seed * 7919 + self.rank)
        scale = init_scale if init_scale is not None else (1.0 / rows) ** 0.5
        self.weight = (torch.rand(rows, self.cols, generator=g, device=self.device) * 2 - 1).mul_(scale).to(dtype)
        self.state = torch.zeros(rows, dtype=torch.float32, device=self.device)
        self.lr, self.eps = lr, eps
        self.comm, self.recv = "nccl", None

    # ------------------------------------------------------------------ the id half
    def input_dist(self, ids: torch.Tensor) -> dict:
        srt = S.sort_unique(ids.reshape(-1), S.key_bits_for(self.rows))
        n_u = srt.n_unique()                                            # the lookup's one host read
        uniq = srt.uniq[:n_u]
        W = self.world
        if W == 1:
            return {"uniq": uniq, "inverse": srt.inverse, "srt": srt, "req_ids": uniq, "counts": [n_u]}
        mine = torch.tensor([n_u], dtype=torch.int64, device=uniq.device)
        allc = [torch.empty_like(mine) for _ in range(W)]
        dist.all_gather(allc, mine, group=self.group)
        counts = torch.cat(allc).tolist()
        req_ids = torch.empty(sum(counts), dtype=torch.int64, device=uniq.device)
        dist.all_to_all_single(req_ids, uniq.repeat(W), counts, [n_u] * W, group=self.group)
        return {"uniq": uniq, "inverse": srt.inverse, "srt": srt, "req_ids": req_ids, "counts": counts}

    def _forward_rows(self, ids, plan: dict | None = None):
        plan = plan if plan is not None else self.input_dist(ids)
        uniq, req_ids, counts = plan["uniq"], plan["req_ids"], plan["counts"]
        W, n_u = self.world, plan["uniq"].numel()
        served = K.gather_rows(self.weight, req_ids)                    # my columns of every rank's rows
        if W == 1:
            rows_u = served
        else:
            got = torch.empty((W * n_u, self.cols), dtype=self.weight.dtype, device=served.device)
            dist.all_to_all_single(got, served, [n_u] * W, counts, group=self.group)
            rows_u = got.view(W, n_u, self.cols).transpose(0, 1).reshape(n_u, self.dim)
        return rows_u, (uniq, plan["inverse"], req_ids, counts, None, plan["srt"])

    def _backward_rows(self, grad: torch.Tensor, ctx_state) -> None:
        uniq, _inverse, req_ids, counts, _, srt = ctx_state
        W, n_u = self.world, uniq.numel()
        wire = torch.bfloat16 if self.weight.dtype == torch.bfloat16 else torch.float32
        if grad.dtype not in (torch.bfloat16, torch.float32):
            grad = grad.float()
        g_u = S.segment_sum(grad, srt, out_dtype=wire if W > 1 else torch.float32, max_seg=n_u)
        if W == 1:
            self.apply_rowwise_adagrad(req_ids, g_u)
            return
        send = g_u.view(n_u, W, self.cols).transpose(0, 1).contiguous().view(W * n_u, self.cols)
        recv = torch.empty((sum(counts), self.cols), dtype=wire, device=grad.device)
        dist.all_to_all_single(recv, send, counts, [n_u] * W, group=self.group)
        srt_l = S.sort_unique(req_ids, S.key_bits_for(max(self.rows, 2)))
        g_l = S.segment_sum(recv, srt_l, out_dtype=torch.float32)
        self.apply_rowwise_adagrad(srt_l.uniq, g_l)

    # ------------------------------------------------------------------ state
    def state_dict(self) -> dict:
        key = f"embeddings.{self.name}.weight"
        return {key: self.weight, f"{key}.col_offset": self.col_lo, f"{key}.global_cols": self.dim,
                f"embeddings.{self.name}.rowwise_adagrad.sum": self.state}

    def load_state_dict(self, sd: dict) -> None:
        key = f"embeddings.{self.name}.weight"
        if int(sd[f"{key}.col_offset"]) != self.col_lo or int(sd[f"{key}.global_cols"]) != self.dim:
            raise ValueError("embedding shard layout differs from the checkpoint (resharding is not supported here)")
        self.weight.copy_(sd[key])
        self.state.copy_(sd[f"embeddings.{self.name}.rowwise_adagrad.sum"])

    def sharded_state_dict(self, prefix: str = "") -> dict:
        """The table as a ``ShardedTensor`` cut along columns (readable under any other placement); the Adagrad
        sums as ``[rows, W]``, one column per shard - they only reload under the same number of ranks."""
        from torch.distributed._shard.sharded_tensor import Shard, ShardMetadata, init_from_local_shards
        wkey, skey = f"{prefix}embeddings.{self.name}.weight", f"{prefix}embeddings.{self.name}.rowwise_adagrad.sum"
        if self.world == 1:
            return {wkey: self.weight, skey: self.state}
        owner = self.rank if (self.group is None or self.group is dist.group.WORLD) else dist.get_global_rank(self.group, self.rank)
        dev = f"rank:{owner}/{'cpu' if self.device.type == 'cpu' else str(self.device)}"
        w = Shard(tensor=self.weight, metadata=ShardMetadata(shard_offsets=[0, self.col_lo], shard_sizes=list(self.weight.shape), placement=dev))
        s = Shard(tensor=self.state.view(self.rows, 1), metadata=ShardMetadata(shard_offsets=[0, self.rank], shard_sizes=[self.rows, 1], placement=dev))
        return {wkey: init_from_local_shards([w], self.rows, self.dim, process_group=self.group),
                skey: init_from_local_shards([s], self.rows, self.world, process_group=self.group)}
