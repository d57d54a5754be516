"""Mixture-of-experts operators: router top-k, device-side dispatch plan, row permutation and
grouped expert GEMMs, with autograd.

Everything that depends on the routing result (per-expert counts, padded segment offsets, the
expert of every 128-row tile, destination rows) stays on the device; the only host-visible size is
the static upper bound ``max_rows(T * k, E)`` of the padded buffer.  This is the property the
reference's "sync-free MoE stage" and ``host_sync_free.py`` work for
(small_llm_moe_pretraining/primus/config_MI355X_1x8x1_tp1pp1ep1_gbs32.sh:156,
generative_recommenders/dlrm_v4/host_sync_free.py).

Router semantics: fp32 logits, top-k, softmax over the selected logits, no auxiliary loss, no
capacity / token dropping (small_llm_moe_pretraining/primus/conf/gpt_oss_20B-MXFP4-deosc-mlperf-pretrain.yaml:115-118,130-167).
"""
from __future__ import annotations

import torch
from torch.autograd import Function

from . import kernels as K
from . import mxfp8
from ._lib import call, ptr, stream_ptr, use_kernels

PAD = 128        # row padding of an expert segment for the bf16 grouped kernels (one 128-row tile)
PAD_MX = 256     # ... for the block-scaled grouped kernels (one CTA pair works on 256 rows)


def pad_rows(precision: str) -> int:
    """Segment padding the grouped kernels of ``precision`` need."""
    from .linear import is_mx
    return PAD_MX if is_mx(precision) else PAD


def grouped_bn(n: int) -> int:
    """N tile of the block-scaled grouped GEMM for a per-expert output width ``n`` (0 = unsupported width)."""
    from . import _lib
    if _lib.LIB_PATH.exists():
        return int(_lib.load().b200_gemm_grouped_mx_bn(int(n)))
    return 192 if n % 192 == 0 else (128 if n % 128 == 0 else 0)


def mx_supported(w1: torch.Tensor, w2: torch.Tensor) -> bool:
    """Whether the expert weights ``w1 [E, 2F, D]`` / ``w2 [E, D, F]`` fit the block-scaled grouped kernels."""
    _, f2, d = w1.shape
    f = w2.shape[2]
    return all(grouped_bn(n) > 0 for n in (f2, d, f)) and d % 32 == 0 and f % 32 == 0


def max_rows(pairs: int, n_experts: int, pad: int = PAD) -> int:
    """Static upper bound of the padded, expert-grouped buffer for ``pairs`` (token, slot) pairs."""
    return (pairs + n_experts * (pad - 1) + pad - 1) // pad * pad


# --------------------------------------------------------------------------------------
# raw ops
# --------------------------------------------------------------------------------------
def router_topk(logits: torch.Tensor, k: int):
    """``logits`` fp32 ``[T, E]`` -> ``(idx int32 [T,k], w fp32 [T,k], counts int32 [E])``."""
    T, E = logits.shape
    if not use_kernels(logits):
        val, idx = torch.topk(logits.float(), k, dim=-1)
        w = torch.softmax(val, dim=-1)
        counts = torch.bincount(idx.reshape(-1), minlength=E).to(torch.int32)
        return idx.to(torch.int32), w, counts
    logits = logits.float().contiguous()
    idx = torch.empty((T, k), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    counts = torch.zeros(E, dtype=torch.int32, device=logits.device)
    call("b200_router_topk", ptr(logits), T, E, k, ptr(idx), ptr(w), ptr(counts), stream_ptr())
    return idx, w, counts


def plan(idx: torch.Tensor, counts: torch.Tensor, n_experts: int, pad: int = PAD):
    """Dispatch plan from the routing result: ``seg [E+1]`` padded segment offsets, ``tile_expert
    [rows/pad]`` (-1 past the end), ``dest [pairs]`` destination row of every (token, slot) pair in
    flattened order (stable inside an expert), ``rows`` the static buffer height."""
    pairs = idx.numel()
    rows = max_rows(pairs, n_experts, pad)
    n_tiles = rows // pad
    if not use_kernels(idx):
        padded = (counts.long() + pad - 1) // pad * pad
        seg = torch.zeros(n_experts + 1, dtype=torch.int64)
        seg[1:] = torch.cumsum(padded, 0)
        flat = idx.reshape(-1).long()
        order = torch.argsort(flat, stable=True)
        rank_in = torch.empty(pairs, dtype=torch.int64)
        sorted_e = flat[order]
        start = torch.zeros(n_experts + 1, dtype=torch.int64)
        start[1:] = torch.cumsum(counts.long(), 0)
        rank_in[order] = torch.arange(pairs) - start[sorted_e]
        dest = (seg[flat] + rank_in).to(torch.int32)
        tile_start = torch.arange(n_tiles) * pad
        te = torch.searchsorted(seg[1:], tile_start, right=True)
        te = torch.where(tile_start < seg[-1], te, torch.full_like(te, -1)).to(torch.int32)
        return seg.to(torch.int32), te, dest, rows
    dev = idx.device
    seg = torch.empty(n_experts + 1, dtype=torch.int32, device=dev)
    te = torch.empty(n_tiles, dtype=torch.int32, device=dev)
    dest = torch.empty(pairs, dtype=torch.int32, device=dev)
    call("b200_router_plan", ptr(counts), ptr(idx.contiguous()), pairs, n_experts, pad, ptr(seg), ptr(te), n_tiles,
         ptr(dest), stream_ptr())
    return seg, te, dest, rows


def permute_rows(x: torch.Tensor, dest: torch.Tensor, k: int, rows: int) -> torch.Tensor:
    """``out[dest[p]] = x[p // k]``; rows that no pair maps to are zero."""
    T, D = x.shape
    out = torch.zeros((rows, D), dtype=x.dtype, device=x.device)
    if not use_kernels(x) or x.dtype != torch.bfloat16:
        out[dest.long()] = x.repeat_interleave(k, dim=0)
        return out
    call("b200_permute_rows", ptr(x.contiguous()), ptr(dest), dest.numel(), k, D, ptr(out), None, None, stream_ptr())
    return out


def unpermute_sum(yp: torch.Tensor, dest: torch.Tensor, w: torch.Tensor | None, T: int, k: int) -> torch.Tensor:
    """``y[t] = sum_j w[t,j] * yp[dest[t*k + j]]`` (``w`` None = plain sum)."""
    D = yp.shape[1]
    if not use_kernels(yp) or yp.dtype != torch.bfloat16:
        g = yp[dest.long()].view(T, k, D).float()
        if w is not None:
            g = g * w.view(T, k, 1).float()
        return g.sum(1).to(yp.dtype)
    y = torch.empty((T, D), dtype=yp.dtype, device=yp.device)
    wf = None if w is None else w.float().contiguous()
    call("b200_unpermute_sum", ptr(yp.contiguous()), ptr(dest), ptr(wf), T, k, D, ptr(y), stream_ptr())
    return y


def grouped_rows(a: torch.Tensor, b: torch.Tensor, tile_expert: torch.Tensor, seg: torch.Tensor, *,
                 b_mn_major: bool = False, out: torch.Tensor | None = None) -> torch.Tensor:
    """``d[r] = a[r] @ op(b[e(r)])^T`` over the padded row buffer.  ``b`` is ``[E, N, K]`` or, with
    ``b_mn_major``, ``[E, K, N]``.  ``out``: write the result there (a peer-visible slab) instead of a new tensor."""
    rows, Kd = a.shape
    E = b.shape[0]
    N = b.shape[2] if b_mn_major else b.shape[1]
    if not use_kernels(a) or a.dtype != torch.bfloat16:
        out = torch.zeros((rows, N), dtype=a.dtype, device=a.device) if out is None else out.zero_()
        s = seg.tolist()
        for e in range(E):
            if s[e + 1] > s[e]:
                w = b[e].float() if b_mn_major else b[e].float().t()
                out[s[e]:s[e + 1]] = (a[s[e]:s[e + 1]].float() @ w).to(a.dtype)
        return out
    if out is None:
        out = torch.empty((rows, N), dtype=a.dtype, device=a.device)
    call("b200_gemm_grouped_rows", ptr(a.contiguous()), ptr(b.contiguous()), ptr(out), ptr(tile_expert), rows, N, Kd, E,
         a.stride(0), out.stride(0), int(b_mn_major), 0, 1.0, stream_ptr())
    # tiles past the last segment are not written: their rows are padding and are never read back
    return out


def grouped_wgrad(dy: torch.Tensor, x: torch.Tensor, seg: torch.Tensor, n_experts: int, *,
                  out: torch.Tensor | None = None, accumulate: bool = False, out_dtype=None) -> torch.Tensor:
    """``d[e] (+)= dy[seg[e]:seg[e+1]]^T @ x[seg[e]:seg[e+1]]`` -> ``[E, M, N]``."""
    M, N = dy.shape[1], x.shape[1]
    if out is None:
        out = torch.zeros((n_experts, M, N), dtype=out_dtype or dy.dtype, device=dy.device)
        accumulate = True if use_kernels(dy) else accumulate
    if not use_kernels(dy) or dy.dtype != torch.bfloat16:
        s = seg.tolist()
        for e in range(n_experts):
            g = dy[s[e]:s[e + 1]].float().t() @ x[s[e]:s[e + 1]].float()
            if accumulate:
                out[e] += g.to(out.dtype)
            else:
                out[e] = g.to(out.dtype)
        return out
    call("b200_gemm_grouped_wgrad", ptr(dy.contiguous()), ptr(x.contiguous()), ptr(out), ptr(seg), dy.shape[0], M, N,
         n_experts, dy.stride(0), x.stride(0), int(out.dtype == torch.float32), int(accumulate), 1.0, stream_ptr())
    return out


# --------------------------------------------------------------------------------------
# autograd
# --------------------------------------------------------------------------------------
class RouterFn(Function):
    """top-k + softmax over the selected logits; the gradient flows to the selected logits only."""

    @staticmethod
    def forward(ctx, logits, k):
        idx, w, counts = router_topk(logits, k)
        ctx.save_for_backward(idx, w)
        ctx.shape = logits.shape
        ctx.mark_non_differentiable(idx, counts)
        return idx, w, counts

    @staticmethod
    def backward(ctx, _gidx, gw, _gc):
        idx, w = ctx.saved_tensors
        g = w * (gw - (w * gw).sum(-1, keepdim=True))
        out = torch.zeros(ctx.shape, dtype=gw.dtype, device=gw.device)
        out.scatter_(1, idx.long(), g)
        return out, None


class PermuteFn(Function):
    @staticmethod
    def forward(ctx, x, dest, k, rows):
        ctx.save_for_backward(dest)
        ctx.cfg = (x.shape[0], k)
        return permute_rows(x, dest, k, rows)

    @staticmethod
    def backward(ctx, g):
        (dest,) = ctx.saved_tensors
        T, k = ctx.cfg
        return unpermute_sum(g.contiguous(), dest, None, T, k), None, None, None


class UnpermuteFn(Function):
    @staticmethod
    def forward(ctx, yp, dest, w, T, k):
        ctx.save_for_backward(yp, dest, w)
        ctx.cfg = (T, k)
        return unpermute_sum(yp, dest, w, T, k)

    @staticmethod
    def backward(ctx, gy):
        yp, dest, w = ctx.saved_tensors
        T, k = ctx.cfg
        D = yp.shape[1]
        gy = gy.contiguous()
        if use_kernels(gy) and gy.dtype == torch.bfloat16 and yp.dtype == torch.bfloat16:
            # one pass: scaled scatter of the gradient rows and the routing-weight gradient (a dot product per pair)
            gyp = torch.zeros_like(yp)
            gw32 = None if w is None else torch.empty(T * k, dtype=torch.float32, device=gy.device)
            wf = None if w is None else w.reshape(-1).float().contiguous()
            call("b200_unpermute_bwd", ptr(gy), ptr(yp.contiguous()), ptr(dest), ptr(wf), T * k, k, D, ptr(gyp), ptr(gw32),
                 stream_ptr())
            return gyp, None, (None if w is None else gw32.view(T, k).to(w.dtype)), None, None
        gyp = permute_rows(gy, dest, k, yp.shape[0])
        gw = None
        if w is not None:
            # scale the scattered rows by their routing weight; weight gradient = <gy[t], yp[dest]>
            scale = torch.zeros(yp.shape[0], dtype=torch.float32, device=yp.device)
            scale[dest.long()] = w.reshape(-1).float()
            gw = (yp[dest.long()].view(T, k, D).float() * gy.view(T, 1, D).float()).sum(-1).to(w.dtype)
            gyp = (gyp.float() * scale[:, None]).to(gyp.dtype)
        return gyp, None, gw, None, None


class GroupedMLPFn(Function):
    """Expert MLP over the padded row buffer: ``swiglu(x W1[e]^T) W2[e]^T`` with the activation
    recomputed in backward.  ``w1`` ``[E, 2F, D]`` (gate rows first), ``w2`` ``[E, D, F]``.  Weight
    gradients accumulate into ``main_grad`` when the parameters carry one."""

    @staticmethod
    def forward(ctx, x, w1, w2, seg, tile_expert, y_out=None, dx_out=None):
        gu = grouped_rows(x, w1, tile_expert, seg)
        a = K.swiglu_fwd(gu)
        y = grouped_rows(a, w2, tile_expert, seg, out=y_out)
        ctx.save_for_backward(x, gu, w1, w2, seg, tile_expert)
        ctx.refs = (w1, w2)
        ctx.dx_out = dx_out
        return y

    @staticmethod
    def backward(ctx, gy):
        x, gu, w1, w2, seg, tile_expert = ctx.saved_tensors
        p1, p2 = ctx.refs
        E = w1.shape[0]
        gy = _zero_padding(gy.contiguous(), tile_expert)
        a = K.swiglu_fwd(gu)
        a = _zero_padding(a, tile_expert)
        g2 = _wgrad_into(p2, gy, a, seg, E)
        da = grouped_rows(gy, w2, tile_expert, seg, b_mn_major=True)
        dgu = K.swiglu_bwd(da, gu)
        dgu = _zero_padding(dgu, tile_expert)
        g1 = _wgrad_into(p1, dgu, x, seg, E)
        dx = grouped_rows(dgu, w1, tile_expert, seg, b_mn_major=True, out=ctx.dx_out)
        return dx, g1, g2, None, None, None, None


# --------------------------------------------------------------------------------------
# block-scaled (MXFP8) expert MLP
# --------------------------------------------------------------------------------------
def _stacked_weight_op(w: torch.Tensor, transposed: bool, fmt: str = "e4m3") -> mxfp8.MXOperand:
    """Quantised copy of the stacked expert weight ``w [E, N, K]`` (or of every expert's transpose) as one
    K-major operand of ``E * N`` rows, scale tiles of ``grouped_bn(N)`` rows, elements of format ``fmt``; cached until
    the weight changes."""
    from .linear import weight_epoch
    key = "_mx_stack_t" if transposed else "_mx_stack"
    hit = getattr(w, key, None)
    stamp = (w._version, weight_epoch(), fmt)
    if hit is not None and hit[0] == stamp:
        return hit[1]
    src = w.detach().transpose(1, 2).contiguous() if transposed else w.detach()
    E, N, Kd = src.shape
    op, _ = mxfp8.quantize(src.reshape(E * N, Kd), row_tile=grouped_bn(N), fmt=fmt)
    setattr(w, key, (stamp, op))
    return op


def grouped_rows_mx(a: mxfp8.MXOperand, b: mxfp8.MXOperand, tile_expert: torch.Tensor, n_experts: int,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """``d[r] = deq(a)[r] @ deq(b)[e(r) * N : (e(r) + 1) * N]^T`` -> bf16 ``[rows, N]``; ``tile_expert`` names the
    expert of every 256-row tile (-1: not computed, rows left unwritten)."""
    rows, Kd = a.rows, a.k
    N = b.rows // n_experts
    if not a.is_cuda:
        A, B = mxfp8.dequantize(a), mxfp8.dequantize(b).view(n_experts, N, Kd)
        out = torch.zeros((rows, N), dtype=torch.bfloat16) if out is None else out.zero_()
        for t, e in enumerate(tile_expert.tolist()):
            if e >= 0:
                out[t * PAD_MX:(t + 1) * PAD_MX] = (A[t * PAD_MX:(t + 1) * PAD_MX] @ B[e].t()).to(torch.bfloat16)
        return out
    if out is None:
        out = torch.empty((rows, N), dtype=torch.bfloat16, device=a.q.device)
    call("b200_gemm_grouped_mx_rows", ptr(a.q), ptr(a.sf), ptr(b.q), ptr(b.sf), ptr(out), ptr(tile_expert), rows, N, Kd,
         n_experts, a.q.stride(0), b.q.stride(0), out.stride(0), 0, 1.0, stream_ptr())
    return out


def grouped_wgrad_mx(dy_t: mxfp8.MXOperand, x_t: mxfp8.MXOperand, seg: torch.Tensor, n_experts: int, out: torch.Tensor):
    """``out[e] += deq(dy_t)[:, seg[e]:seg[e+1]] @ deq(x_t)[:, seg[e]:seg[e+1]]^T``; both operands are column-wise
    copies (rows = features, contraction = the padded buffer's rows); ``out`` ``[E, M, N]`` fp32 or bf16."""
    M, N, T = dy_t.rows, x_t.rows, dy_t.k
    if not dy_t.is_cuda:
        A, B = mxfp8.dequantize(dy_t), mxfp8.dequantize(x_t)
        s = seg.tolist()
        for e in range(n_experts):
            out[e] += (A[:, s[e]:s[e + 1]] @ B[:, s[e]:s[e + 1]].t()).to(out.dtype)
        return out
    call("b200_gemm_grouped_mx_wgrad", ptr(dy_t.q), ptr(dy_t.sf), ptr(x_t.q), ptr(x_t.sf), ptr(out), ptr(seg), T, M, N,
         n_experts, dy_t.q.stride(0), x_t.q.stride(0), int(out.dtype == torch.float32), 1, 1.0, stream_ptr())
    return out


class GroupedMLPMXFn(Function):
    """``GroupedMLPFn`` with every GEMM on block-scaled e4m3 operands: the row buffer is quantised once per
    use (row-wise copy for the forward / dgrad GEMM, column-wise copy for the weight gradient), SwiGLU and
    its backward are folded into the quantiser where the width allows, the stacked weights are quantised once
    per optimizer step.  Expert segments start at multiples of 256 rows."""

    @staticmethod
    def forward(ctx, x, w1, w2, seg, tile_expert, y_out=None, dx_out=None, recipe="mxfp8"):
        from .linear import MX_RECIPES
        E, F2, D = w1.shape
        F = F2 // 2
        f_act, f_w, _, _, b_act, _, _ = MX_RECIPES[recipe]
        narrow = recipe != "mxfp8"
        if narrow:
            x = _zero_padding_mx(x, tile_expert)
        x_row, x_col = mxfp8.quantize(x, row_tile=mxfp8.A_TILE, col_tile=grouped_bn(D), fmt=f_act, col_fmt=b_act)
        # rows of tiles past the last segment are never written and never contribute: the row GEMMs skip those
        # tiles and the weight-gradient contraction stops at the last segment's end
        gu = grouped_rows_mx(x_row, _stacked_weight_op(w1, False, f_w), tile_expert, E)
        if narrow:            # the fused SwiGLU quantiser writes e4m3 elements: the narrow formats round a materialised activation
            a_row, a_col = mxfp8.quantize(_zero_padding_mx(K.swiglu_fwd(gu), tile_expert), row_tile=mxfp8.A_TILE,
                                          col_tile=grouped_bn(F), fmt=f_act, col_fmt=b_act)
        else:
            a_row, a_col = mxfp8.quantize_swiglu(gu, row_tile=mxfp8.A_TILE, col_tile=grouped_bn(F))
        y = grouped_rows_mx(a_row, _stacked_weight_op(w2, False, f_w), tile_expert, E, out=y_out)
        ctx.save_for_backward(gu, w1, w2, seg, tile_expert, x_col.q, x_col.sf, a_col.q, a_col.sf)
        ctx.refs = (w1, w2)
        ctx.dx_out = dx_out
        ctx.dims = (x.shape[0], D, F)
        ctx.recipe = recipe
        return y

    @staticmethod
    def backward(ctx, gy):
        from .linear import MX_RECIPES
        gu, w1, w2, seg, tile_expert, xq, xsf, aq, asf = ctx.saved_tensors
        p1, p2 = ctx.refs
        rows, D, F = ctx.dims
        E = w1.shape[0]
        _, _, g_fmt, b_w, _, g_sr, _ = MX_RECIPES[ctx.recipe]
        narrow = ctx.recipe != "mxfp8"
        x_col = mxfp8.MXOperand(xq, xsf, D, rows, grouped_bn(D))
        a_col = mxfp8.MXOperand(aq, asf, F, rows, grouped_bn(F))
        gy = gy.contiguous()
        if narrow:
            gy = _zero_padding_mx(gy, tile_expert)
        gy_row, gy_col = mxfp8.quantize(gy, row_tile=mxfp8.A_TILE, col_tile=mxfp8.A_TILE, fmt=g_fmt, stochastic=g_sr)
        g2 = _wgrad_into_mx(p2, gy_col, a_col, seg, E)
        da = grouped_rows_mx(gy_row, _stacked_weight_op(w2, True, b_w), tile_expert, E)
        if narrow:
            dgu_row, dgu_col = mxfp8.quantize(_zero_padding_mx(K.swiglu_bwd(da, gu), tile_expert), row_tile=mxfp8.A_TILE,
                                              col_tile=mxfp8.A_TILE, fmt=g_fmt, stochastic=g_sr)
        else:
            dgu_row, dgu_col = mxfp8.quantize_swiglu_bwd(da, gu, row_tile=mxfp8.A_TILE, col_tile=mxfp8.A_TILE)
        g1 = _wgrad_into_mx(p1, dgu_col, x_col, seg, E)
        dx = grouped_rows_mx(dgu_row, _stacked_weight_op(w1, True, b_w), tile_expert, E, out=ctx.dx_out)
        return dx, g1, g2, None, None, None, None, None


def _zero_padding_mx(t: torch.Tensor, tile_expert: torch.Tensor) -> torch.Tensor:
    """Rows of 256-row tiles without an expert are never written by the grouped GEMM and may hold anything (NaN
    included); the tensor-operation quantiser of the narrow formats reads whole 32-row blocks, so clear them first."""
    dead = (tile_expert < 0).repeat_interleave(PAD_MX)
    if dead.numel() != t.shape[0]:
        return t
    return t.masked_fill(dead[:, None], 0)


def _wgrad_into_mx(param, dy_t, x_t, seg, E):
    if not param.requires_grad:
        return None
    mg = getattr(param, "main_grad", None)
    if mg is not None:
        grouped_wgrad_mx(dy_t, x_t, seg, E, mg)
        return None
    out = torch.zeros((E, dy_t.rows, x_t.rows), dtype=torch.float32, device=dy_t.q.device)
    return grouped_wgrad_mx(dy_t, x_t, seg, E, out).to(param.dtype)


def grouped_mlp(x, w1, w2, seg, tile_expert, precision: str = "bf16", y_out=None, dx_out=None):
    """Expert MLP over a padded row buffer whose segments are padded to ``pad_rows(precision)``.  ``y_out`` /
    ``dx_out``: buffers of the row buffer's shape that receive the output / the input gradient (peer-visible slabs
    of the expert-parallel dispatch, filled by the last GEMM of each direction instead of by a copy)."""
    from .linear import is_mx
    if is_mx(precision):
        return GroupedMLPMXFn.apply(x, w1, w2, seg, tile_expert, y_out, dx_out, precision)
    return GroupedMLPFn.apply(x, w1, w2, seg, tile_expert, y_out, dx_out)


def _zero_padding(t: torch.Tensor, tile_expert: torch.Tensor) -> torch.Tensor:
    """Rows of tiles past the last segment may hold stale memory: zero them so the weight-gradient
    contraction over whole tiles is exact (rows inside a segment's padding are already zero because
    they come from zero inputs)."""
    if tile_expert.numel() * PAD != t.shape[0]:
        return t
    if use_kernels(t) and t.dtype == torch.bfloat16 and t.is_contiguous():
        call("b200_zero_dead_tiles", ptr(t), ptr(tile_expert), tile_expert.numel(), t.shape[1], stream_ptr())   # in place
        return t
    dead = (tile_expert < 0).repeat_interleave(PAD)
    return t.masked_fill(dead[:, None], 0)


def _wgrad_into(param, dy, x, seg, E):
    mg = getattr(param, "main_grad", None)
    if not param.requires_grad:
        return None
    if mg is not None:
        grouped_wgrad(dy, x, seg, E, out=mg, accumulate=True)
        return None
    return grouped_wgrad(dy, x, seg, E, out_dtype=param.dtype)


def expert_precision(precision: str, w1, w2) -> str:
    """Precision the expert GEMMs run at: the micro-scaled recipe asked for when the widths fit the block-scaled
    grouped tiles, else bf16."""
    from .linear import is_mx
    if is_mx(precision) and w1.dtype == torch.bfloat16 and mx_supported(w1, w2):
        return precision
    return "bf16"


def moe_experts(x, idx, w, counts, w1, w2, precision: str = "bf16"):
    """Local (all experts on this rank) MoE expert stage: dispatch by permutation, grouped MLP,
    weighted combine.  ``x`` ``[T, D]``; returns ``[T, D]``."""
    T, k = idx.shape
    E = w1.shape[0]
    precision = expert_precision(precision, w1, w2)
    seg, tile_expert, dest, rows = plan(idx, counts, E, pad=pad_rows(precision))
    xp = PermuteFn.apply(x, dest, k, rows)
    yp = grouped_mlp(xp, w1, w2, seg, tile_expert, precision)
    return UnpermuteFn.apply(yp, dest, w, T, k)
