"""Tensor parallelism with sequence parallelism (Megatron layout) over 2-D ``[tokens, features]``
activations.

Between the tensor-parallel regions an activation is sharded along tokens (rank ``r`` of ``W``
holds rows ``[r*T/W, (r+1)*T/W)``); inside a region it is sharded along features:

* ``column_parallel(x_shard, w_local)``  all-gather(x) -> ``x_full @ w_local^T`` : ``[T, N/W]``;
  backward: dgrad ``dy @ w_local`` reduce-scattered to ``[T/W, K]``, wgrad ``dy^T x_full``.
* ``row_parallel(x, w_local, residual_shard)``  ``x @ w_local^T`` is a partial sum, reduce-scattered
  (+ residual) to ``[T/W, N]``; backward: all-gather(dy) -> dgrad ``dy_full @ w_local``, wgrad
  ``dy_full^T x``.

``comm="nccl"`` runs the collectives through ``torch.distributed`` around the plain GEMM (the
structure of the reference, where the userbuffer overlap is off:
llama2_sft/primus/config_MI355X_1x8x1.sh:115-118; llama2_sft/primus/conf/llama2_70b_lora_posttrain.yaml:18-23).
``comm="fused"`` uses the all-gather->GEMM and GEMM->reduce-scatter kernels of ``csrc/gemm_tp.cu``:
the transfer happens inside the GEMM kernel over peer memory, tile by tile.

Weight gradients are accumulated into ``weight.main_grad`` when the parameter has one.

``precision="fp8"`` (fused path, frozen weights - the base of a LoRA run): the weight is quantised once to
per-tensor e4m3 (both orientations), activations go to e4m3 and gradients to e5m2 with delayed scaling, and
the fused kernels run the 8-bit tensor-core path; gathered blocks cross NVLink as codes, one byte per
element.  A gathered tensor is decoded with ONE factor, so its sites share their scale across the group:
their amax words live in one pool that is max-reduced over the group once per optimizer step
(llama2_sft/primus/src/llama2_custom.py:1904-1910 pre-quantises the frozen base in the reference).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist
from torch.autograd import Function

from ..ops import _lib
from ..ops import fp8 as F8
from ..ops import kernels as K
from ..ops.functional import _wgrad
from ..ops.linear import _site, fp8_weight_operands, weight_epoch


class TPContext:
    RS_FLAG_OFFSET = 64     # ints: [0, 16) all-gather block counters, [64, ...) reduce-scatter tile counters

    def __init__(self, group=None, comm: str = "nccl", device=None, n_copy: int = 0, n_red: int = 8, copy_mode: int = 1,
                 precision: str = "bf16"):
        self.group = group
        self.precision = precision      # "fp8": frozen-weight linears of the fused path run on 8-bit operands
        self._amax_pool = None          # int32 words of the sites whose scale is shared by the group
        self._amax_used = 0
        self._amax_epoch = None
        on = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if on else 1
        self.rank = dist.get_rank(group) if on else 0
        self.device = torch.device(device) if device is not None else None
        self.comm = comm
        # copy CTAs of the all-gather kernel: enough to move (W-1)/W of the operand within the GEMM's time
        self.n_copy = n_copy if n_copy > 0 else (16 if self.world >= 4 else 8)
        self.n_red, self.copy_mode = n_red, copy_mode
        self._gather = [None, None]     # double-buffered symmetric gather buffers
        self._gather_turn = 0
        self._stage = None
        self._flags = None              # symmetric int32 counters (reduce-scatter), zeroed before each use
        self._local_flags = None        # local int32: [0:16] chunk flags, [16] work counter

    # ------------------------------------------------------------------ plain collectives
    def all_gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return x
        x = x.contiguous()
        out = torch.empty((x.shape[0] * self.world, *x.shape[1:]), dtype=x.dtype, device=x.device)
        if x.is_cuda:
            dist.all_gather_into_tensor(out, x, group=self.group)
        else:
            dist.all_gather(list(out.chunk(self.world, 0)), x, group=self.group)
        return out

    def reduce_scatter_rows(self, y: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return y
        y = y.contiguous()
        rows = y.shape[0] // self.world
        if y.is_cuda:
            out = torch.empty((rows, *y.shape[1:]), dtype=y.dtype, device=y.device)
            dist.reduce_scatter_tensor(out, y, group=self.group)
            return out
        dist.all_reduce(y, group=self.group)
        return y[self.rank * rows:(self.rank + 1) * rows].clone()

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return t

    # ------------------------------------------------------------------ fused-path resources
    def fused_ok(self, t: torch.Tensor) -> bool:
        return self.comm == "fused" and t.is_cuda and t.dtype == torch.bfloat16

    def fp8_ok(self, t: torch.Tensor, weight: torch.Tensor) -> bool:
        """8-bit path: fused kernels, a frozen bf16 weight, every dimension a multiple of 128."""
        return (self.precision == "fp8" and self.fused_ok(t) and not weight.requires_grad and weight.dtype == torch.bfloat16
                and t.shape[0] % 128 == 0 and t.shape[1] % 128 == 0 and weight.shape[0] % 128 == 0 and weight.shape[1] % 128 == 0)

    def shared_site(self, weight: torch.Tensor, name: str, fmt: str) -> "F8.DelayedScale":
        """Scale state of a tensor that is gathered over the group: its amax word is a slot of the pool."""
        st = _site(weight, name, fmt)
        if getattr(st, "_pooled", None) is not self:
            if self._amax_pool is None:
                self._amax_pool = torch.zeros(8192, dtype=torch.int32, device=weight.device)
            if self._amax_used >= self._amax_pool.numel():
                raise RuntimeError("tensor-parallel FP8: more shared scale sites than pool slots")
            st.amax = self._amax_pool[self._amax_used:self._amax_used + 1]
            self._amax_used += 1
            st._pooled = self
        return st

    def prepare_shared(self, st: "F8.DelayedScale", x: torch.Tensor) -> None:
        """``st.scale`` valid for ``x`` in the current epoch and equal on every rank of the group."""
        epoch = weight_epoch()
        if not st.primed:
            a = x.detach().abs().amax().float().reshape(1)
            if self.world > 1:
                dist.all_reduce(a, op=dist.ReduceOp.MAX, group=self.group)
            st._set_from(a)
            st.primed, st.epoch = True, epoch
            return
        if epoch != self._amax_epoch:
            # one max-reduction of every shared site's amax per optimizer step (bit patterns of non-negative
            # floats order like the floats); sites primed in this epoch hold zeros and are not rolled yet
            self._amax_epoch = epoch
            if self.world > 1 and self._amax_used:
                dist.all_reduce(self._amax_pool[: self._amax_used], op=dist.ReduceOp.MAX, group=self.group)
        st.prepare(x, epoch)

    def _symm(self, numel: int, dtype):
        from .symm import SymmetricBuffer
        return SymmetricBuffer(numel, dtype, self.group, self.device)

    def _ensure(self, gather_numel: int = 0, stage_numel: int = 0) -> None:
        """Grow the symmetric buffers (collective: every rank asks for the same sizes in the same order)."""
        if gather_numel and (self._gather[0] is None or self._gather[0].local.numel() < gather_numel):
            self._gather = [self._symm(gather_numel, torch.bfloat16), self._symm(gather_numel, torch.bfloat16)]
        if stage_numel and (self._stage is None or self._stage.local.numel() < stage_numel):
            self._stage = self._symm(stage_numel, torch.bfloat16)
        if self._flags is None:
            self._flags = self._symm(4096, torch.int32)
            self._local_flags = torch.zeros(32, dtype=torch.int32, device=self._flags.local.device)

    def gather_begin(self, x_shard: torch.Tensor):
        """Place this rank's row block into the next gather buffer and synchronise the ranks.
        Returns ``(buffer, full_view [T, K])``; the peers' blocks are filled by the consuming kernel."""
        rows, k = x_shard.shape
        self._ensure(gather_numel=rows * self.world * k)
        buf = self._gather[self._gather_turn]
        self._gather_turn ^= 1
        full = buf.local[: rows * self.world * k].view(rows * self.world, k)
        full[self.rank * rows:(self.rank + 1) * rows].copy_(x_shard)
        self._flags.local.zero_()
        buf.barrier()          # every block is in place and every counter is zero before any rank launches
        return buf, full

    def gather_begin_codes(self, q_shard: torch.Tensor):
        """``gather_begin`` for a block of 8-bit codes ``[rows, k]`` (uint8): the gather buffer is viewed as bytes."""
        rows, k = q_shard.shape
        self._ensure(gather_numel=(rows * self.world * k + 1) // 2)
        buf = self._gather[self._gather_turn]
        self._gather_turn ^= 1
        full = buf.local.view(torch.uint8)[: rows * self.world * k].view(rows * self.world, k)
        full[self.rank * rows:(self.rank + 1) * rows].copy_(q_shard)
        self._flags.local.zero_()
        buf.barrier()
        return buf, full

    def gemm_gather_fp8(self, buf, full: torch.Tensor, a_inv: torch.Tensor, a_fmt: str, b: "F8.FP8Operand") -> torch.Tensor:
        """``dequant(full [T, K] codes) @ dequant(b [N, K])^T -> [T, N]`` bf16, the peers' row blocks of ``full``
        pulled or pushed inside the kernel."""
        W, r = self.world, self.rank
        T, Kd = full.shape
        N = b.rows
        rows_per = T // W
        out = torch.empty((T, N), dtype=torch.bfloat16, device=full.device)
        if rows_per % 256 == 0:
            # the CTA-pair core with copy pairs inside the launch
            _lib.call("b200_gemm_tp_gather_pair", _lib.ptr(full), _lib.ptr(b.q), _lib.ptr(out), T, N, Kd, full.stride(0),
                      b.q.stride(0), out.stride(0), 1, int(a_fmt == "e5m2"), int(b.fmt == "e5m2"), _lib.ptr(a_inv),
                      _lib.ptr(b.inv_scale), 1.0, buf.ptr_array(), W, r, _lib.ptr(full), rows_per * Kd, rows_per,
                      _lib.ptr(self._flags.local), self.n_copy, self.copy_mode, self._flags.ptr_array(), _lib.stream_ptr())
            return out
        _lib.call("b200_gemm_tp_gather_fp8", _lib.ptr(full), _lib.ptr(b.q), _lib.ptr(out), T, N, Kd, full.stride(0),
                  b.q.stride(0), out.stride(0), int(a_fmt == "e5m2"), int(b.fmt == "e5m2"), _lib.ptr(a_inv), _lib.ptr(b.inv_scale),
                  0, 0, 1.0, 1, buf.ptr_array(), W, r, _lib.ptr(full), rows_per * Kd, rows_per, _lib.ptr(self._flags.local),
                  self.n_copy, self.copy_mode, self._flags.ptr_array(), _lib.stream_ptr())
        return out

    def gemm_reduce_scatter_fp8(self, a: "F8.FP8Operand", b: "F8.FP8Operand", residual: torch.Tensor | None = None) -> torch.Tensor:
        """``reduce_scatter_rows(dequant(a) @ dequant(b)^T) (+ residual)`` -> ``[T/W, N]`` bf16 in one kernel."""
        W, r = self.world, self.rank
        M, Kd, N = a.rows, a.k, b.rows
        rows_per = M // W
        self._ensure(stage_numel=M * N)
        self._flags.local.zero_()
        self._local_flags.zero_()
        self._stage.barrier()
        out = torch.empty((rows_per, N), dtype=torch.bfloat16, device=a.q.device)
        if rows_per % 256 == 0:
            _lib.call("b200_gemm_tp_rs_pair", _lib.ptr(a.q), _lib.ptr(b.q), M, N, Kd, a.q.stride(0), b.q.stride(0), 1,
                      int(a.fmt == "e5m2"), int(b.fmt == "e5m2"), _lib.ptr(a.inv_scale), _lib.ptr(b.inv_scale), 1.0,
                      self._stage.ptr_array(), self._flags.offset_ptr_array(4 * self.RS_FLAG_OFFSET), W, r,
                      _lib.ptr(self._local_flags[16:]), _lib.ptr(out), out.stride(0),
                      None if residual is None else _lib.ptr(residual), 0 if residual is None else residual.stride(0), self.n_red,
                      _lib.stream_ptr())
            return out
        _lib.call("b200_gemm_tp_rs_fp8", _lib.ptr(a.q), _lib.ptr(b.q), M, N, Kd, a.q.stride(0), b.q.stride(0),
                  int(a.fmt == "e5m2"), int(b.fmt == "e5m2"), _lib.ptr(a.inv_scale), _lib.ptr(b.inv_scale), 1.0,
                  self._stage.ptr_array(), self._flags.offset_ptr_array(4 * self.RS_FLAG_OFFSET), W, r,
                  _lib.ptr(self._local_flags[16:]), _lib.ptr(out), out.stride(0),
                  None if residual is None else _lib.ptr(residual), 0 if residual is None else residual.stride(0), self.n_red,
                  _lib.stream_ptr())
        return out

    def gemm_gather(self, buf, full: torch.Tensor, other: torch.Tensor, *, mode: int, out: torch.Tensor | None = None,
                    accumulate: bool = False, out_dtype=torch.bfloat16) -> torch.Tensor:
        """mode 1: ``full [T,K] @ other[N,K]^T -> [T,N]``.  mode 2 (wgrad): ``other[T,N]^T @ full[T,K] -> [N,K]``,
        the gathered dimension being the reduction."""
        W, r = self.world, self.rank
        T, Kf = full.shape
        rows_per = T // W
        if mode == 1:
            a, b, M, N, Kd, a_mn, b_mn = full, other, T, other.shape[0], Kf, 0, 0
        else:
            a, b, M, N, Kd, a_mn, b_mn = other, full, other.shape[1], Kf, T, 1, 1
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype, device=full.device)
        if mode == 1 and rows_per % 256 == 0 and out.dtype == torch.bfloat16 and not accumulate:
            # the CTA-pair core with copy pairs inside the launch
            _lib.call("b200_gemm_tp_gather_pair", _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), M, N, Kd, a.stride(0), b.stride(0),
                      out.stride(0), 0, 0, 0, None, None, 1.0, buf.ptr_array(), W, r, _lib.ptr(full), rows_per * Kf * 2, rows_per,
                      _lib.ptr(self._flags.local), self.n_copy, self.copy_mode, self._flags.ptr_array(), _lib.stream_ptr())
            return out
        _lib.call("b200_gemm_tp_gather", _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), M, N, Kd, a.stride(0), b.stride(0),
                  out.stride(0), a_mn, b_mn, int(out.dtype == torch.float32), int(accumulate), 1.0, mode,
                  buf.ptr_array(), W, r, _lib.ptr(full), rows_per * Kf * 2, rows_per, _lib.ptr(self._flags.local),
                  self.n_copy, self.copy_mode, self._flags.ptr_array(), _lib.stream_ptr())
        return out

    def gemm_reduce_scatter(self, a: torch.Tensor, b: torch.Tensor, *, b_mn_major: bool = False,
                            residual: torch.Tensor | None = None) -> torch.Tensor:
        """``reduce_scatter_rows(a @ op(b)^T) (+ residual)`` -> ``[T/W, N]`` bf16 in one kernel."""
        W, r = self.world, self.rank
        M, Kd = a.shape
        N = b.shape[1] if b_mn_major else b.shape[0]
        rows_per = M // W
        self._ensure(stage_numel=M * N)
        self._flags.local.zero_()
        self._local_flags.zero_()
        self._stage.barrier()           # counters are zero everywhere, previous readers of the staging buffer are done
        out = torch.empty((rows_per, N), dtype=torch.bfloat16, device=a.device)
        if rows_per % 256 == 0 and not b_mn_major:
            # the CTA-pair core with reduce pairs inside the launch
            _lib.call("b200_gemm_tp_rs_pair", _lib.ptr(a), _lib.ptr(b), M, N, Kd, a.stride(0), b.stride(0), 0, 0, 0, None, None, 1.0,
                      self._stage.ptr_array(), self._flags.offset_ptr_array(4 * self.RS_FLAG_OFFSET), W, r,
                      _lib.ptr(self._local_flags[16:]), _lib.ptr(out), out.stride(0),
                      None if residual is None else _lib.ptr(residual), 0 if residual is None else residual.stride(0), self.n_red,
                      _lib.stream_ptr())
            return out
        _lib.call("b200_gemm_tp_rs", _lib.ptr(a), _lib.ptr(b), M, N, Kd, a.stride(0), b.stride(0), 0, int(b_mn_major), 1.0,
                  self._stage.ptr_array(), self._flags.offset_ptr_array(4 * self.RS_FLAG_OFFSET), W, r,
                  _lib.ptr(self._local_flags[16:]),
                  _lib.ptr(out), out.stride(0), None if residual is None else _lib.ptr(residual),
                  0 if residual is None else residual.stride(0), self.n_red, _lib.stream_ptr())
        return out


class ColumnParallelFn(Function):
    @staticmethod
    def forward(ctx, x_shard, weight, tp: TPContext):
        ctx.tp = tp
        ctx.fp8 = tp.fp8_ok(x_shard, weight)
        if ctx.fp8:
            # frozen weight: no weight gradient, so the activation is not kept
            ctx.save_for_backward(weight)
            st = tp.shared_site(weight, "x", "e4m3")
            tp.prepare_shared(st, x_shard)
            xq, _ = F8.quantize(x_shard, st)
            buf, full = tp.gather_begin_codes(xq.q)
            w_row, _ = fp8_weight_operands(weight)
            return tp.gemm_gather_fp8(buf, full, st.inv_scale, "e4m3", w_row)
        ctx.save_for_backward(x_shard, weight)
        if tp.fused_ok(x_shard):
            buf, full = tp.gather_begin(x_shard)
            return tp.gemm_gather(buf, full, weight, mode=1)
        return K.gemm(tp.all_gather_rows(x_shard), weight)

    @staticmethod
    def backward(ctx, dy):
        tp: TPContext = ctx.tp
        if ctx.fp8:
            (weight,) = ctx.saved_tensors
            if not ctx.needs_input_grad[0]:
                return None, None, None
            dy = dy.contiguous()
            st = _site(weight, "dy", "e5m2")            # partial sums are decoded per rank: a local scale is enough
            st.prepare(dy, weight_epoch())
            dyq, _ = F8.quantize(dy, st)
            _, w_col = fp8_weight_operands(weight)      # [K, N_local]: contraction over the local output features
            return tp.gemm_reduce_scatter_fp8(dyq, w_col), None, None
        x_shard, weight = ctx.saved_tensors
        dy = dy.contiguous()
        need_w = weight.requires_grad
        if tp.fused_ok(dy):
            dx = tp.gemm_reduce_scatter(dy, weight, b_mn_major=True) if ctx.needs_input_grad[0] else None
            dw = None
            if need_w:
                buf, full = tp.gather_begin(x_shard)
                mg = getattr(weight, "main_grad", None)
                if mg is not None and mg.dtype == torch.float32:
                    tp.gemm_gather(buf, full, dy, mode=2, out=mg, accumulate=True)
                else:
                    dw = tp.gemm_gather(buf, full, dy, mode=2, out_dtype=weight.dtype)
                    if mg is not None:
                        mg.add_(dw.to(mg.dtype))
                        dw = None
            return dx, dw, None
        dx = None
        if ctx.needs_input_grad[0]:
            dx = tp.reduce_scatter_rows(K.gemm(dy, weight, b_mn_major=True))
        dw = _wgrad(dy, tp.all_gather_rows(x_shard), weight) if need_w else None
        return dx, dw, None


class RowParallelFn(Function):
    @staticmethod
    def forward(ctx, x, weight, residual_shard, tp: TPContext):
        ctx.tp = tp
        ctx.has_res = residual_shard is not None
        ctx.fp8 = tp.fp8_ok(x, weight)
        if ctx.fp8:
            ctx.save_for_backward(weight)
            st = _site(weight, "x", "e4m3")
            st.prepare(x, weight_epoch())
            xq, _ = F8.quantize(x.contiguous(), st)
            w_row, _ = fp8_weight_operands(weight)
            return tp.gemm_reduce_scatter_fp8(xq, w_row, residual=residual_shard)
        ctx.save_for_backward(x, weight)
        if tp.fused_ok(x):
            return tp.gemm_reduce_scatter(x.contiguous(), weight, residual=residual_shard)
        y = tp.reduce_scatter_rows(K.gemm(x, weight))
        return y if residual_shard is None else y + residual_shard

    @staticmethod
    def backward(ctx, dy_shard):
        tp: TPContext = ctx.tp
        if ctx.fp8:
            (weight,) = ctx.saved_tensors
            dy_shard = dy_shard.contiguous()
            dx = None
            if ctx.needs_input_grad[0]:
                st = tp.shared_site(weight, "dy", "e5m2")
                tp.prepare_shared(st, dy_shard)
                dyq, _ = F8.quantize(dy_shard, st)
                buf, full = tp.gather_begin_codes(dyq.q)
                _, w_col = fp8_weight_operands(weight)  # [K_local, N]: contraction over the output features
                dx = tp.gemm_gather_fp8(buf, full, st.inv_scale, "e5m2", w_col)
            return dx, None, (dy_shard if ctx.has_res else None), None
        x, weight = ctx.saved_tensors
        dy_shard = dy_shard.contiguous()
        if tp.fused_ok(dy_shard):
            buf, dy_full = tp.gather_begin(dy_shard)
            dx = _gather_dgrad(tp, buf, dy_full, weight)      # also completes dy_full in the local buffer
            dw = _wgrad(dy_full, x, weight) if weight.requires_grad else None    # dy_full is complete after the kernel above
        else:
            dy_full = tp.all_gather_rows(dy_shard)
            dx = K.gemm(dy_full, weight, b_mn_major=True) if ctx.needs_input_grad[0] else None
            dw = _wgrad(dy_full, x, weight) if weight.requires_grad else None
        return dx, dw, (dy_shard if ctx.has_res else None), None


def _gather_dgrad(tp: TPContext, buf, dy_full: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """all-gather(dy) -> ``dy_full @ weight`` with ``weight [N, K_local]`` as the MN-major B operand."""
    W, r = tp.world, tp.rank
    T, N = dy_full.shape
    k_local = weight.shape[1]
    out = torch.empty((T, k_local), dtype=torch.bfloat16, device=dy_full.device)
    _lib.call("b200_gemm_tp_gather", _lib.ptr(dy_full), _lib.ptr(weight), _lib.ptr(out), T, k_local, N, dy_full.stride(0),
              weight.stride(0), out.stride(0), 0, 1, 0, 0, 1.0, 1, buf.ptr_array(), W, r, _lib.ptr(dy_full),
              (T // W) * N * 2, T // W, _lib.ptr(tp._flags.local), tp.n_copy, tp.copy_mode, tp._flags.ptr_array(),
              _lib.stream_ptr())
    return out


def column_parallel(x_shard: torch.Tensor, weight: torch.Tensor, tp: TPContext) -> torch.Tensor:
    return ColumnParallelFn.apply(x_shard, weight, tp)


def row_parallel(x: torch.Tensor, weight: torch.Tensor, tp: TPContext, residual: torch.Tensor | None = None) -> torch.Tensor:
    return RowParallelFn.apply(x, weight, residual, tp)


class CopyToTP(Function):
    """Identity forward, all-reduce backward: marks where a replicated tensor enters per-rank compute."""

    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return x

    @staticmethod
    def backward(ctx, g):
        return ctx.tp.all_reduce(g.contiguous()), None


class ReduceFromTP(Function):
    """All-reduce forward, identity backward."""

    @staticmethod
    def forward(ctx, x, tp):
        return tp.all_reduce(x.contiguous().clone())

    @staticmethod
    def backward(ctx, g):
        return g, None


class GatherRows(Function):
    """all-gather rows forward, take the local row block backward (for tensors whose consumers
    already reduce over ranks) - used by the LoRA side path."""

    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return tp.all_gather_rows(x)

    @staticmethod
    def backward(ctx, g):
        tp = ctx.tp
        return tp.reduce_scatter_rows(g.contiguous()), None


class ScatterRows(Function):
    """reduce-scatter rows forward, all-gather backward."""

    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return tp.reduce_scatter_rows(x.contiguous())

    @staticmethod
    def backward(ctx, g):
        return ctx.tp.all_gather_rows(g.contiguous()), None
