"""Precision-aware GEMM triple of a linear layer (forward, dgrad, wgrad).

``precision="bf16"`` runs the bf16 tcgen05 GEMM on the tensors as they are (the backward GEMMs read
the same row-major buffers as MN-major operands).  ``precision="fp8"`` runs the per-tensor FP8 GEMM
(e4m3 activations and weights, e5m2 gradients, delayed scaling: ``ops.fp8``); the scale state of the
three tensor sites of a linear (input, weight, output gradient) lives on the weight parameter.
``precision="mxfp8"`` runs the block-scaled
GEMM: activations and gradients are quantised on the fly (one pass gives the row-wise copy for the
next GEMM and the transposed column-wise copy that the weight-gradient GEMM needs later), weights
are quantised once per optimizer step in both directions and cached on the parameter.  The narrower
members of the micro-scaled family (``mxfp6``, ``mxfp4``, ``a6w4``: ``MX_RECIPES``) run the same GEMM on
operands whose elements were rounded to the 6- or 4-bit format first - every such value is an e4m3 value, so
the product is the narrow format's, bit for bit, at the 8-bit operand rate; gradients of the 4-bit recipes are
rounded stochastically and their weight-gradient operands pass a block Hadamard transform along the tokens.

What is saved for backward is the return value of ``forward`` (a bf16 tensor or the fp8 operand);
``Saved.pack`` / ``Saved.unpack`` move it through ``ctx.save_for_backward``.

Mirrors the recipe plumbing the reference gets from Transformer Engine (quantised copies of
weights cached between micro-batches, column-wise copies kept for wgrad;
llama2_sft/primus/src/llama2_custom.py:1904-1910 pre-quantises frozen base weights once).
"""
from __future__ import annotations

import torch

from . import fp8 as F8
from . import kernels as K
from . import mxfp8 as MX

# bumped by the optimizer engine after every parameter update: invalidates cached weight copies
_WEIGHT_EPOCH = 0


def weight_epoch() -> int:
    """Counter that advances whenever parameters may have changed outside autograd's version tracking."""
    return _WEIGHT_EPOCH


def bump_weight_epoch() -> None:
    global _WEIGHT_EPOCH
    _WEIGHT_EPOCH += 1


# micro-scaled recipes: element format of (forward activation, forward weight, gradient, backward weight, activation kept
# for the weight gradient), stochastic rounding of the gradient operands, Hadamard block along the tokens for the
# weight-gradient operands (0 = none).  "a6w4": forward in MXFP6 activations x MXFP4 weights, backward in MXFP4
# (flux1/primus/patches/flux_fprop_switch.py:36-120); "mxfp4": llama2_sft/primus/patches/megatron_lm_mxfp4_recipe.patch:66-84.
MX_RECIPES = {
    "mxfp8": ("e4m3", "e4m3", "e4m3", "e4m3", "e4m3", False, 0),
    "mxfp6": ("e2m3", "e2m3", "e3m2", "e2m3", "e2m3", False, 0),
    "mxfp4": ("e2m1", "e2m1", "e2m1", "e2m1", "e2m1", True, 16),
    "a6w4": ("e2m3", "e2m1", "e2m1", "e2m1", "e2m1", True, 16),
    # the phase a FLUX run switches to: forward at 8 bits, backward still at 4
    "mxfp8_fwd_mxfp4_bwd": ("e4m3", "e4m3", "e2m1", "e2m1", "e2m1", True, 16),
}


def is_mx(precision: str) -> bool:
    return precision in MX_RECIPES


_HADAMARD: dict = {}


def hadamard_rows(x: torch.Tensor, block: int) -> torch.Tensor:
    """``x [T, C]`` with every group of ``block`` consecutive rows multiplied by the orthonormal Hadamard matrix of that
    size: ``hadamard_rows(a).T @ hadamard_rows(b) == a.T @ b`` exactly in real arithmetic, while outliers of a column are
    spread over the block before the operands are rounded."""
    key = (block, x.device, x.dtype)
    h = _HADAMARD.get(key)
    if h is None:
        h = torch.ones(1, 1)
        while h.shape[0] < block:
            h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
        h = _HADAMARD[key] = (h / block ** 0.5).to(device=x.device, dtype=x.dtype)
    T, C = x.shape
    return torch.matmul(h, x.reshape(T // block, block, C)).reshape(T, C)


def mx_eligible(rows: int, n_out: int, n_in: int) -> bool:
    """MXFP8 needs every GEMM dimension to be a multiple of 128 (tokens, out and in features)."""
    return rows % 128 == 0 and n_out % 128 == 0 and n_in % 128 == 0


def weight_operands(weight: torch.Tensor, need_col: bool = True, fmt: str = "e4m3", col_fmt: str | None = None):
    """(w_row, w_col) micro-scaled copies of ``weight`` ``[N, K]``: ``w_row`` (rows N, contraction K) is
    the B operand of forward, ``w_col`` (rows K, contraction N) the B operand of dgrad.  Cached on
    the tensor until the next optimizer step (or forever for frozen weights); ``fmt`` / ``col_fmt``: their element
    formats (part of the cache key)."""
    cache = getattr(weight, "_mx_cache", None)
    col_fmt = col_fmt or fmt
    epoch = (_WEIGHT_EPOCH if weight.requires_grad else -1, fmt, col_fmt)
    if cache is not None and cache[0] == epoch and (cache[2] is not None or not need_col):
        return cache[1], cache[2]
    N, Kd = weight.shape
    w = weight.detach()
    if w.dtype != torch.bfloat16 and w.is_cuda:
        w = w.to(torch.bfloat16)
    row, col = MX.quantize(w, row_tile=MX.b_tile(N), col_tile=MX.b_tile(Kd) if need_col else None, fmt=fmt, col_fmt=col_fmt)
    weight._mx_cache = (epoch, row, col)
    return row, col


def _site(weight: torch.Tensor, name: str, fmt: str) -> "F8.DelayedScale":
    """Delayed-scaling state of one tensor site of the linear that owns ``weight``."""
    sites = getattr(weight, "_fp8_sites", None)
    if sites is None:
        sites = weight._fp8_sites = {}
    st = sites.get(name)
    if st is None or st.fmt != fmt:
        st = sites[name] = F8.DelayedScale(fmt, weight.device)
    return st


def fp8_weight_operands(weight: torch.Tensor, need_col: bool = True):
    """(w_row, w_col) per-tensor e4m3 copies of ``weight [N, K]`` (``w_col`` is the transposed copy for
    dgrad), cached until the next optimizer step."""
    cache = getattr(weight, "_fp8_cache", None)
    epoch = _WEIGHT_EPOCH if weight.requires_grad else -1
    if cache is not None and cache[0] == epoch and (cache[2] is not None or not need_col):
        return cache[1], cache[2]
    w = weight.detach()
    if w.dtype != torch.bfloat16 and w.is_cuda:
        w = w.to(torch.bfloat16)
    st = _site(weight, "w", "e4m3")
    st.prepare(w, epoch)
    row, col = F8.quantize(w, st, want_row=True, want_col=need_col)
    weight._fp8_cache = (epoch, row, col)
    return row, col


class Saved:
    """The activation copy kept for the weight-gradient GEMM."""

    @staticmethod
    def pack(obj):
        if isinstance(obj, MX.MXOperand):
            return [obj.q, obj.sf], ("mx", obj.rows, obj.k, obj.tile_rows)
        if isinstance(obj, F8.FP8Operand):
            return [obj.q, obj.inv_scale], ("f8", obj.rows, obj.k, obj.fmt)
        return [obj], ("t",)

    @staticmethod
    def unpack(tensors, meta):
        if meta[0] == "mx":
            return MX.MXOperand(tensors[0], tensors[1], meta[1], meta[2], meta[3])
        if meta[0] == "f8":
            return F8.FP8Operand(tensors[0], tensors[1], meta[1], meta[2], meta[3])
        return tensors[0]


def low_precision(precision: str, rows: int, n_out: int, n_in: int) -> bool:
    """The call runs a quantised GEMM (and saves a quantised activation copy for backward)."""
    # (the per-tensor FP8 GEMM has CTA-pair tiles only: its M - the tokens in forward and dgrad, the output
    # features in wgrad - must exceed one 128-row tile)
    return (is_mx(precision) or precision == "fp8") and mx_eligible(rows, n_out, n_in) and (is_mx(precision) or (rows > 128 and n_out > 128))


def forward(x: torch.Tensor, weight: torch.Tensor, precision: str, *, bias=None, residual=None,
            need_wgrad: bool = True):
    """``y = x W^T (+ bias) (+ residual)``.  Returns ``(y, saved)`` where ``saved`` is what
    ``backward`` needs of ``x`` (None when ``need_wgrad`` is False)."""
    M, Kd = x.shape
    N = weight.shape[0]
    if is_mx(precision) and mx_eligible(M, N, Kd):
        f_act, f_w, _, b_w, b_act, _, had = MX_RECIPES[precision]
        w_row, _ = weight_operands(weight, need_col=False, fmt=f_w, col_fmt=b_w)
        if had and need_wgrad and M % had == 0:
            # the copy kept for the weight gradient passes the Hadamard transform along the tokens (its partner, the
            # output gradient, gets the same one in backward)
            x_row, _ = MX.quantize(x, row_tile=MX.A_TILE, fmt=f_act)
            _, x_col = MX.quantize(hadamard_rows(x, had), col_tile=MX.b_tile(Kd), fmt=b_act)
        else:
            x_row, x_col = MX.quantize(x, row_tile=MX.A_TILE, col_tile=MX.b_tile(Kd) if need_wgrad else None, fmt=f_act,
                                       col_fmt=b_act)
        y = MX.gemm(x_row, w_row, bias=bias, residual=residual, out_dtype=x.dtype)
        return y, x_col
    if precision == "fp8" and low_precision(precision, M, N, Kd):
        w_row, _ = fp8_weight_operands(weight, need_col=False)
        st = _site(weight, "x", "e4m3")
        st.prepare(x, _WEIGHT_EPOCH)
        x_row, x_col = F8.quantize(x, st, want_row=True, want_col=need_wgrad)
        y = F8.gemm(x_row, w_row, bias=bias, residual=residual, out_dtype=x.dtype)
        return y, x_col
    y = K.gemm(x, weight, bias=bias, residual=residual)
    return y, (x if need_wgrad else None)


def backward(dy: torch.Tensor, saved, weight: torch.Tensor, precision: str, *, need_dx: bool = True,
             need_dw: bool = True):
    """Returns ``(dx, dw)``.  ``dw`` is None when it was accumulated into ``weight.main_grad``
    (or not requested)."""
    M, N = dy.shape
    Kd = weight.shape[1]
    dx = dw = None
    use_mx = is_mx(precision) and mx_eligible(M, N, Kd)
    if use_mx:
        _, f_w, g_fmt, b_w, b_act, g_sr, had = MX_RECIPES[precision]
        had = had if M % max(had, 1) == 0 else 0
    if use_mx and need_dw and not isinstance(saved, MX.MXOperand):
        # the forward ran in bf16 for this call (e.g. recomputed activation): quantise now
        _, saved = MX.quantize(hadamard_rows(saved, had) if had else saved, col_tile=MX.b_tile(Kd), fmt=b_act)
    if use_mx:
        if had and need_dw:
            dy_row = MX.quantize(dy, row_tile=MX.A_TILE, fmt=g_fmt, stochastic=g_sr)[0] if need_dx else None
            _, dy_col = MX.quantize(hadamard_rows(dy, had), col_tile=MX.A_TILE, fmt=g_fmt, stochastic=g_sr)
        else:
            dy_row, dy_col = MX.quantize(dy, row_tile=MX.A_TILE if need_dx else None,
                                         col_tile=MX.A_TILE if need_dw else None, fmt=g_fmt, stochastic=g_sr)
        if need_dx:
            _, w_col = weight_operands(weight, need_col=True, fmt=f_w, col_fmt=b_w)
            dx = MX.gemm(dy_row, w_col, out_dtype=dy.dtype)
        if need_dw:
            mg = getattr(weight, "main_grad", None)
            if mg is not None:
                MX.gemm(dy_col, saved, out=mg, accumulate=True)
            else:
                dw = MX.gemm(dy_col, saved, out_dtype=weight.dtype if weight.dtype != torch.float32 else torch.float32)
        return dx, dw
    if precision == "fp8" and low_precision(precision, M, N, Kd):
        if need_dw and not isinstance(saved, F8.FP8Operand):
            st = _site(weight, "x", "e4m3")
            st.prepare(saved, _WEIGHT_EPOCH)
            _, saved = F8.quantize(saved, st, want_row=False, want_col=True)
        st = _site(weight, "dy", "e5m2")                 # gradients: e5m2 (range over precision)
        st.prepare(dy, _WEIGHT_EPOCH)
        dy_row, dy_col = F8.quantize(dy, st, want_row=need_dx, want_col=need_dw)
        if need_dx:
            _, w_col = fp8_weight_operands(weight, need_col=True)
            dx = F8.gemm(dy_row, w_col, out_dtype=dy.dtype)
        if need_dw:
            mg = getattr(weight, "main_grad", None)
            if mg is not None:
                F8.gemm(dy_col, saved, out=mg, accumulate=True)
            else:
                dw = F8.gemm(dy_col, saved, out_dtype=weight.dtype if weight.dtype != torch.float32 else torch.float32)
        return dx, dw
    if isinstance(saved, F8.FP8Operand):
        # the forward ran in fp8 but this backward cannot (a dimension of 128): dequantise the saved copy
        saved = F8.dequantize(saved).t().contiguous().to(dy.dtype)
    if need_dx:
        dx = K.gemm(dy, weight, b_mn_major=True)
    if need_dw:
        mg = getattr(weight, "main_grad", None)
        if mg is not None:
            K.gemm(dy, saved, a_mn_major=True, b_mn_major=True, out=mg, accumulate=True)
        else:
            dw = K.gemm(dy, saved, a_mn_major=True, b_mn_major=True, out_dtype=weight.dtype)
    return dx, dw
