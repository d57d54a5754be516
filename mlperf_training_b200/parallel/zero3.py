"""Sharded-parameter (ZeRO-3 / FSDP) engine: the matrices of every transformer block live as 1/W
shards; a block's full parameters exist only while the block computes, in one of two rotating
windows, and its gradients leave the window for the owners' fp32 shard accumulators as soon as the
block's backward has finished.

Layout per block bucket (``block0007``: the block's matrices; its vectors - norm weights, sinks -
stay replicated in a small ZeRO-1 bucket ``block0007_v``, and so do the embedding, the head and the
final norm):

* ``param_buf``  this rank's bf16 shard (``numel / W`` elements), the persistent copy;
* ``grad_buf``   this rank's fp32 gradient shard, accumulated over micro-batches;
* ``m, v``       Adam moments of the shard;
* window slot ``block_index % 2``: full-size bf16 parameter window and fp32 gradient window that the
  block's parameter tensors (``p.data``, ``p.main_grad``) are views of.

Schedule (hooks called by the model around every block):

* ``pre_forward(i)``   waits for the gather of block i, then starts the gather of block i + 1 into the
  other slot on the communication stream (it overlaps block i's compute);
* ``pre_backward(i)``  waits for block i's parameters (re-gathered unless still resident) and for its
  gradient window to be free, then starts the gather of block i - 1;
* ``post_backward(i)`` reduce-scatters the gradient window into ``grad_buf`` (+=) on the
  communication stream and clears the window.

With MXFP8 linears the quantised weight copies are cached on the parameters until the optimizer
step, so after the first micro-batch of a step a block's gather is skipped whenever every matrix
of the block still has its cached copies (the gathered bf16 values would not be read).

Transports: NCCL / gloo collectives; or, on symmetric windows bound to an NVLink multicast object,
this package's NVLS kernels (``multimem.st`` all-gather, ``multimem.ld_reduce`` reduce-scatter:
csrc/fused_zero.cu) between cross-rank barriers.

Reference behaviour covered: torch FSDP2 local-shard wrappers with forward prefetch and (optional)
resharding after forward as configured for FLUX (flux1/primus/patches/flux_fprop_switch.py:114-194,
flux1/primus/conf/flux.1_schnell_t2i-pretrain.yaml:48-49,71) and Megatron's overlapped parameter
gather (small_llm_pretraining/primus/conf/llama3.1_8B-pretrain-fp4.yaml:54-60).
"""
from __future__ import annotations

import os
import re

import torch
import torch.distributed as dist

from ..ops import kernels as K
from ..ops import linear as L
from .engine import OptimConfig, ZeroEngine, default_bucket_of


class Zero3Engine(ZeroEngine):
    def __init__(self, model, opt: OptimConfig, *, group=None, comm: str = "nccl", skip_cached: bool = True):
        self._vec_names: set[str] = {n for n, p in model.named_parameters() if p.dim() < 2}

        def bucket_of(name: str) -> str:
            key = default_bucket_of(name)
            return key + "_v" if (key.startswith("block") and name in self._vec_names) else key

        # the replicated buckets (vectors, embedding, head) take the library collectives of the base engine
        super().__init__(model, opt, group=group, bucket_of=bucket_of, comm="nccl")
        self.z3_comm = comm
        self.skip_cached = skip_cached
        self.blocks3 = [b for b in self.buckets if re.fullmatch(r"block\d+", b.key) and self.world > 1]
        for b in self.buckets:
            b.zero3 = False
        self._stream = None
        self._resident = [None, None]            # (block index, weight epoch) whose parameters a window slot holds
        self._gather_ev = [None, None]
        self._gw_free_ev = [None, None]
        self._rs_pending: list = []
        self._dirty: set[int] = set()            # blocks whose gradient window holds unreduced gradients
        self.win_p = self.win_g = None
        self.nvls = False
        if self.blocks3:
            self._shard_blocks()
        if model is not None and hasattr(model, "block_hooks"):
            model.block_hooks = self if self.blocks3 else None

    # ------------------------------------------------------------------ construction
    def _shard_blocks(self) -> None:
        dev = self.device
        dtype = self.blocks3[0].param_buf.dtype
        n_max = max(b.numel for b in self.blocks3)
        cuda = dev.type == "cuda"
        fused = self.z3_comm == "fused" and cuda and os.environ.get("B200_NVLS", "1") != "0"
        if fused:
            from .symm import SymmetricBuffer
            grp = self.group if self.group is not None else dist.group.WORLD
            self._symm_p = [SymmetricBuffer(n_max, dtype, grp, dev) for _ in range(2)]
            self._symm_g = [SymmetricBuffer(n_max, torch.float32, grp, dev) for _ in range(2)]
            self.nvls = all(s.multicast_ptr != 0 for s in self._symm_p + self._symm_g)
            self.win_p = [s.local for s in self._symm_p]
            self.win_g = [s.local for s in self._symm_g]
        else:
            self.win_p = [torch.zeros(n_max, dtype=dtype, device=dev) for _ in range(2)]
            self.win_g = [torch.zeros(n_max, dtype=torch.float32, device=dev) for _ in range(2)]
        for w in self.win_p + self.win_g:
            w.zero_()
        for b in self.blocks3:
            idx = int(b.key[5:])
            b.zero3, b.block_idx, b.slot = True, idx, idx % 2
            store = b.param_buf[b.lo:b.hi].clone()
            wp, wg = self.win_p[b.slot], self.win_g[b.slot]
            for (name, p), o in zip(b.params, b.offsets):
                n = p.numel()
                p.data = wp[o:o + n].view(p.shape)
                p.main_grad = wg[o:o + n].view(p.shape)
            b.param_buf = store                                   # the persistent copy is the shard
            b.grad_buf = torch.zeros(b.shard, dtype=torch.float32, device=dev)
            b.symm_param = b.symm_grad = None
            if b.master is not None:
                b.master = store.float()
        self._by_block3 = {b.block_idx: b for b in self.blocks3}
        # the matrices are no longer reduced by the base engine's overlap path
        for k in list(self._by_block):
            self._by_block[k] = [b for b in self._by_block[k] if not b.zero3]
        if cuda:
            self._stream = torch.cuda.Stream(device=dev)
            torch.cuda.empty_cache()

    # shard views of a sharded bucket are the buffers themselves
    @staticmethod
    def _ps(b):
        return b.param_buf if b.zero3 else b.p_shard()

    @staticmethod
    def _gs(b):
        return b.grad_buf if b.zero3 else b.g_shard()

    def state_bytes(self) -> int:
        tot = 0
        for b in self.buckets:
            tot += b.param_buf.numel() * b.param_buf.element_size() + b.grad_buf.numel() * b.grad_buf.element_size()
            tot += b.m.numel() * b.m.element_size() + b.v.numel() * b.v.element_size()
        for w in (self.win_p or []) + (self.win_g or []):
            tot += w.numel() * w.element_size()
        return tot

    # ------------------------------------------------------------------ transports
    def _on_comm(self):
        return torch.cuda.stream(self._stream) if self._stream is not None else _Null()

    def _gather(self, b) -> None:
        """All ranks' shards of ``b`` -> window slot (on the communication stream)."""
        win = self.win_p[b.slot][:b.numel]
        if self.nvls:
            from ..ops import _lib
            sp = self._symm_p[b.slot]
            sp.barrier()                                  # every rank has finished reading the slot's previous tenant
            es = b.param_buf.element_size()
            _lib.call("b200_mc_all_gather", _lib.ptr(b.param_buf), sp.multicast_ptr + b.lo * es, b.shard * es, _lib.stream_ptr())
            sp.barrier()                                  # every rank's shard has landed everywhere
        elif dist.get_backend(self.group) == "gloo":
            parts = [torch.empty_like(b.param_buf) for _ in range(self.world)]
            dist.all_gather(parts, b.param_buf, group=self.group)
            win.copy_(torch.cat(parts))
        else:
            dist.all_gather_into_tensor(win, b.param_buf, group=self.group)

    def _reduce(self, b) -> None:
        """Gradient window of ``b`` -> += owners' fp32 shards, mean over ranks; then the window is cleared."""
        win = self.win_g[b.slot][:b.numel]
        if self.nvls:
            from ..ops import _lib
            sg = self._symm_g[b.slot]
            sg.barrier()                                  # every rank's gradients of this block are final
            _lib.call("b200_zero_reduce_scatter_mc", sg.multicast_ptr, b.lo, b.shard, 1.0 / self.world, _lib.ptr(b.grad_buf), 1,
                      None, _lib.stream_ptr())
            sg.barrier()                                  # every owner has read its shard: the windows may be cleared
        elif dist.get_backend(self.group) == "gloo":
            dist.all_reduce(win, group=self.group)
            b.grad_buf.add_(win[b.lo:b.hi], alpha=1.0 / self.world)
        else:
            tmp = torch.empty(b.shard, dtype=torch.float32, device=self.device)
            dist.reduce_scatter_tensor(tmp, win, op=dist.ReduceOp.AVG, group=self.group)
            b.grad_buf.add_(tmp)
        win.zero_()

    # ------------------------------------------------------------------ residency
    def _cached(self, b, need_col: bool) -> bool:
        if not self.skip_cached:
            return False
        for _, p in b.params:
            c = getattr(p, "_mx_cache", None)
            epoch = L._WEIGHT_EPOCH if p.requires_grad else -1
            if c is None or c[0][0] != epoch or (need_col and c[2] is None):      # key: (epoch, row format, column format)
                return False
        return True

    def _ensure(self, idx: int, need_col: bool, prefetch: bool) -> None:
        b = self._by_block3.get(idx)
        if b is None:
            return
        tag = (idx, L._WEIGHT_EPOCH)
        if self._resident[b.slot] == tag or self._cached(b, need_col):
            return
        cur = torch.cuda.current_stream() if self._stream is not None else None
        if self._stream is not None:
            self._stream.wait_stream(cur)                 # the slot's previous tenant has been consumed in stream order
        with self._on_comm():
            self._gather(b)
            if self._stream is not None:
                ev = torch.cuda.Event()
                ev.record(self._stream)
                self._gather_ev[b.slot] = ev
        self._resident[b.slot] = tag
        if not prefetch:
            self._wait_gather(b.slot)

    def _wait_gather(self, slot: int) -> None:
        ev = self._gather_ev[slot]
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
            self._gather_ev[slot] = None

    # ------------------------------------------------------------------ hooks (called by the model)
    def pre_forward(self, idx: int) -> None:
        b = self._by_block3.get(idx)
        if b is None:
            return
        self._ensure(idx, need_col=False, prefetch=False)
        self._wait_gather(b.slot)
        self._ensure(idx + 1, need_col=False, prefetch=True)

    def pre_backward(self, idx: int) -> None:
        b = self._by_block3.get(idx)
        if b is None:
            return
        self._ensure(idx, need_col=True, prefetch=False)
        self._wait_gather(b.slot)
        self._dirty.add(idx)
        ev = self._gw_free_ev[b.slot]
        if ev is not None:                                # the slot's gradient window has been reduced and cleared
            torch.cuda.current_stream().wait_event(ev)
            self._gw_free_ev[b.slot] = None
        self._ensure(idx - 1, need_col=True, prefetch=True)

    def post_backward(self, idx: int) -> None:
        b = self._by_block3.get(idx)
        if b is None or idx not in self._dirty:
            return
        self._dirty.discard(idx)
        if self._stream is not None:
            self._stream.wait_stream(torch.cuda.current_stream())
        with self._on_comm():
            self._reduce(b)
            if self._stream is not None:
                ev = torch.cuda.Event()
                ev.record(self._stream)
                self._gw_free_ev[b.slot] = ev
                self._rs_pending.append(ev)

    # ------------------------------------------------------------------ step
    def zero_grad(self) -> None:
        super().zero_grad()
        for w in self.win_g or []:
            w.zero_()

    @torch.no_grad()
    def step(self, lr: float | None = None, grad_scale: float = 1.0) -> None:
        if not self.blocks3:
            return super().step(lr, grad_scale)
        o = self.opt
        lr = o.lr if lr is None else lr
        self.step_count += 1
        for idx in sorted(self._dirty, reverse=True):     # a block whose input carried no gradient (frozen embedding)
            self.post_backward(idx)
        for ev in self._rs_pending:
            torch.cuda.current_stream().wait_event(ev)
        self._rs_pending.clear()
        early = self._finish_overlap()
        order = list(reversed(self.buckets))
        for b in order:
            if not b.zero3 and id(b) not in early:
                self._reduce_scatter(b)
        clip = o.clip_grad > 0
        if clip:
            first = True
            for b in order:
                K.sumsq(self._gs(b), self.sumsq, accumulate=not first)
                first = False
            dist.all_reduce(self.sumsq, group=self.group)
            self.last_grad_norm = self.sumsq
        for b in order:
            ps, gs = self._ps(b), self._gs(b)
            for s, e, wd in b.segments():
                K.adamw_(ps[s:e], gs[s:e], b.m[s:e], b.v[s:e], lr=lr, beta1=o.beta1, beta2=o.beta2, eps=o.eps,
                         weight_decay=o.weight_decay if wd else 0.0, step=self.step_count,
                         master=None if b.master is None else b.master[s:e], grad_scale=grad_scale,
                         sumsq_buf=self.sumsq if clip else None, max_norm=o.clip_grad, zero_grad=True)
            if not b.zero3 and not getattr(b, "local_only", False):
                if b.lo > 0:
                    b.grad_buf[:b.lo].zero_()
                if b.hi < b.numel:
                    b.grad_buf[b.hi:].zero_()
                self._all_gather(b)
        L.bump_weight_epoch()                             # cached low-precision copies and window contents are stale
        self._resident = [None, None]

    @torch.no_grad()
    def replica_checksum_spread(self) -> float:
        keep = self.buckets
        try:
            self.buckets = [b for b in keep if not b.zero3]     # shards have no replica to be compared with
            return super().replica_checksum_spread()
        finally:
            self.buckets = keep

    @torch.no_grad()
    def gather_full(self, b) -> torch.Tensor:
        """The whole parameter buffer of a sharded bucket (collective; for export and tests)."""
        parts = [torch.empty_like(b.param_buf) for _ in range(self.world)]
        dist.all_gather(parts, b.param_buf.contiguous(), group=self.group)
        return torch.cat(parts)


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False
