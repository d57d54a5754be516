"""Autograd layer over the raw operators of ``ops.kernels``.

Every Function works on 2-D ``[tokens, features]`` activations.  Weight gradients follow the
"gradient accumulation fusion" convention of the reference's Megatron configs
(small_llm_pretraining/primus/conf/llama3.1_8B-pretrain-fp4.yaml:59-61): when a parameter
carries a ``main_grad`` tensor (fp32 or bf16 view into the flat gradient buffer of the
optimizer / FSDP engine), the wgrad GEMM adds straight into it from its epilogue and autograd
receives no gradient for that parameter.
"""
from __future__ import annotations

import math

import torch
from torch.autograd import Function

from . import kernels as K
from . import linear as L
from ._lib import call, ptr, stream_ptr, use_kernels


def _wgrad(dy: torch.Tensor, x: torch.Tensor, weight: torch.Tensor):
    """dW = dy^T x, accumulated into ``weight.main_grad`` when present (returns None then)."""
    if not weight.requires_grad:
        return None
    mg = getattr(weight, "main_grad", None)
    if mg is not None:
        K.gemm(dy, x, a_mn_major=True, b_mn_major=True, out=mg, accumulate=True)
        if hasattr(weight, "grad_added_to_main_grad"):
            weight.grad_added_to_main_grad = True
        return None
    return K.gemm(dy, x, a_mn_major=True, b_mn_major=True, out_dtype=weight.dtype)


def _vec_grad(param: torch.Tensor | None, g: torch.Tensor | None):
    """Route a small (norm weight / bias) gradient to main_grad when present."""
    if param is None or g is None or not param.requires_grad:
        return None
    mg = getattr(param, "main_grad", None)
    if mg is not None:
        mg.add_(g.to(mg.dtype))
        return None
    return g.to(param.dtype)


class LinearFn(Function):
    """y = x W^T (+ bias) (+ residual), the residual add done in the GEMM epilogue."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual, precision):
        need_w = weight.requires_grad
        y, saved = L.forward(x, weight, precision, bias=bias, residual=residual, need_wgrad=need_w)
        tensors, ctx.meta = L.Saved.pack(saved) if saved is not None else ([], None)
        ctx.save_for_backward(weight, *tensors)
        ctx.has_res = residual is not None
        ctx.bias_ref = bias
        ctx.precision = precision
        return y

    @staticmethod
    def backward(ctx, dy):
        weight, *tensors = ctx.saved_tensors
        saved = L.Saved.unpack(tensors, ctx.meta) if ctx.meta is not None else None
        dy = dy.contiguous()
        dx, dw = L.backward(dy, saved, weight, ctx.precision, need_dx=ctx.needs_input_grad[0],
                            need_dw=weight.requires_grad and saved is not None)
        db = _vec_grad(ctx.bias_ref, dy.sum(0, dtype=torch.float32)) if ctx.bias_ref is not None else None
        dres = dy if ctx.has_res and ctx.needs_input_grad[3] else None
        return dx, dw, db, dres, None


def linear(x, weight, bias=None, residual=None, precision="bf16"):
    return LinearFn.apply(x, weight, bias, residual, precision)


class NormFn(Function):
    """RMSNorm / LayerNorm / SwishLayerNorm on rows."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps, layer_norm, swish):
        y, h, mean, rstd = K.norm_fwd(x, weight, bias, eps, layer_norm=layer_norm, swish=swish)
        ctx.save_for_backward(x, weight, bias, mean, rstd)
        ctx.cfg = (layer_norm, swish)
        ctx.refs = (weight, bias)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, bias, mean, rstd = ctx.saved_tensors
        layer_norm, swish = ctx.cfg
        dx, dw, db = K.norm_bwd(dy.contiguous(), x, weight, bias, mean, rstd, layer_norm=layer_norm, swish=swish)
        return dx, _vec_grad(ctx.refs[0], dw), _vec_grad(ctx.refs[1], db), None, None, None


def rms_norm(x, weight, eps=1e-5):
    return NormFn.apply(x, weight, None, eps, False, False)


def layer_norm(x, weight, bias, eps=1e-5):
    return NormFn.apply(x, weight, bias, eps, True, False)


def swish_layer_norm(x, weight, bias, eps=1e-5):
    return NormFn.apply(x, weight, bias, eps, True, True)


class NormLinearFn(Function):
    """y = norm(x) W^T.  bf16: the normalised activation is recomputed in backward instead of saved
    (the "fused residual + RMSNorm -> GEMM" pairing of the reference's Turbo configs,
    small_llm_pretraining/primus/config_MI355X_1x8x1.sh:42-51).  mxfp8: its transposed fp8 copy,
    produced by the same quantisation pass that feeds the forward GEMM, is kept instead."""

    @staticmethod
    def forward(ctx, x, norm_w, norm_b, weight, bias, eps, layer_norm, precision):
        xn, _, mean, rstd = K.norm_fwd(x, norm_w, norm_b, eps, layer_norm=layer_norm)
        keep = L.low_precision(precision, x.shape[0], weight.shape[0], weight.shape[1])
        y, saved = L.forward(xn, weight, precision, bias=bias, need_wgrad=keep and weight.requires_grad)
        tensors, ctx.meta = L.Saved.pack(saved) if saved is not None else ([], None)
        ctx.save_for_backward(x, norm_w, norm_b, weight, mean, rstd, *tensors)
        ctx.cfg = (eps, layer_norm, precision)
        ctx.refs = (norm_w, norm_b, bias)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, norm_w, norm_b, weight, mean, rstd, *tensors = ctx.saved_tensors
        eps, layer_norm, precision = ctx.cfg
        dy = dy.contiguous()
        if ctx.meta is not None:
            saved = L.Saved.unpack(tensors, ctx.meta)
        elif weight.requires_grad:
            saved = K.norm_fwd(x, norm_w, norm_b, eps, layer_norm=layer_norm)[0]
        else:
            saved = None
        dxn, dw = L.backward(dy, saved, weight, precision, need_dx=True,
                             need_dw=weight.requires_grad and saved is not None)
        del saved
        dx, dnw, dnb = K.norm_bwd(dxn, x, norm_w, norm_b, mean, rstd, layer_norm=layer_norm)
        db = _vec_grad(ctx.refs[2], dy.sum(0, dtype=torch.float32)) if ctx.refs[2] is not None else None
        return dx, _vec_grad(ctx.refs[0], dnw), _vec_grad(ctx.refs[1], dnb), dw, db, None, None, None


def norm_linear(x, norm_w, weight, *, norm_b=None, bias=None, eps=1e-5, layer_norm=False, precision="bf16"):
    return NormLinearFn.apply(x, norm_w, norm_b, weight, bias, eps, layer_norm, precision)


class SwiGLULinearFn(Function):
    """out = swiglu(gu) W^T + residual, saving only ``gu`` (the activation is recomputed)."""

    @staticmethod
    def forward(ctx, gu, weight, residual, precision):
        a = K.swiglu_fwd(gu)
        out, _ = L.forward(a, weight, precision, residual=residual, need_wgrad=False)
        ctx.save_for_backward(gu, weight)
        ctx.has_res = residual is not None
        ctx.precision = precision
        return out

    @staticmethod
    def backward(ctx, dy):
        gu, weight = ctx.saved_tensors
        dy = dy.contiguous()
        a = K.swiglu_fwd(gu) if weight.requires_grad else None
        da, dw = L.backward(dy, a, weight, ctx.precision, need_dx=True, need_dw=weight.requires_grad)
        del a
        dgu = K.swiglu_bwd(da, gu)
        return dgu, dw, (dy if ctx.has_res else None), None


def swiglu_linear(gu, weight, residual=None, precision="bf16"):
    return SwiGLULinearFn.apply(gu, weight, residual, precision)


def _mx_wgrad(weight, dy_col, x_col):
    """dW = dy^T x from the transposed MXFP8 copies, into ``main_grad`` when the parameter has one."""
    from . import mxfp8 as MX
    if not weight.requires_grad:
        return None
    mg = getattr(weight, "main_grad", None)
    if mg is not None:
        MX.gemm(dy_col, x_col, out=mg, accumulate=True)
        return None
    return MX.gemm(dy_col, x_col, out_dtype=weight.dtype)


class FusedMLPFn(Function):
    """RMSNorm -> gate/up GEMM -> SwiGLU -> down GEMM (+ residual) as one MXFP8 unit.

    The activation ``a = silu(gate) * up`` and its gradient ``dgu`` never exist in bf16: the
    quantiser computes them on the fly (``quantize_swiglu`` / ``quantize_swiglu_bwd``) and writes only
    the e4m3 copies the GEMMs read.  Saved for backward: the block input, the normalisation
    statistics, ``gu`` and the transposed fp8 copy of the normalised input.  This is the reference's
    fused dense MLP with the quantisation and dGLU folded in
    (small_llm_pretraining/primus/config_MI355X_1x8x1.sh:42-51).

    ``store_fp8``: ``gu`` - the largest saved activation, ``[T, 2F]`` - is kept for backward as per-tensor e4m3
    codes (delayed scale) instead of bf16, half the bytes; backward decodes it before dSwiGLU (the reference's
    SwiGLU op with FP8 input store, llama2_sft/primus/patches/megatron_lm_mxfp4_recipe.patch)."""

    @staticmethod
    def forward(ctx, h, norm_w, w_gu, w_down, eps, store_fp8=False):
        from . import mxfp8 as MX
        D = h.shape[1]
        xn, _, mean, rstd = K.norm_fwd(h, norm_w, None, eps, layer_norm=False)
        need1 = w_gu.requires_grad
        w1_row, _ = L.weight_operands(w_gu, need_col=False)
        xn_row, xn_col = MX.quantize(xn, row_tile=MX.A_TILE, col_tile=MX.b_tile(D) if need1 else None)
        del xn
        gu = MX.gemm(xn_row, w1_row, out_dtype=h.dtype)
        a_row, _ = MX.quantize_swiglu(gu, row_tile=MX.A_TILE)
        w2_row, _ = L.weight_operands(w_down, need_col=False)
        out = MX.gemm(a_row, w2_row, residual=h, out_dtype=h.dtype)
        tensors, ctx.meta = L.Saved.pack(xn_col) if xn_col is not None else ([], None)
        ctx.gu_fp8 = bool(store_fp8)
        if store_fp8:
            from . import fp8 as F8
            st = L._site(w_gu, "gu_store", "e4m3")
            st.prepare(gu, L.weight_epoch())
            op = F8.quantize_rows(gu, st)
            ctx.save_for_backward(h, norm_w, w_gu, w_down, mean, rstd, op.q, op.inv_scale.clone(), *tensors)
        else:
            ctx.save_for_backward(h, norm_w, w_gu, w_down, mean, rstd, gu, *tensors)
        ctx.eps = eps
        ctx.refs = (norm_w, w_gu, w_down)
        return out

    @staticmethod
    def backward(ctx, dy):
        from . import mxfp8 as MX
        if ctx.gu_fp8:
            h, norm_w, w_gu, w_down, mean, rstd, gu_q, gu_inv, *tensors = ctx.saved_tensors
            gu = (gu_q.view(torch.float8_e4m3fn).to(torch.float32) * gu_inv).to(h.dtype)
            del gu_q
        else:
            h, norm_w, w_gu, w_down, mean, rstd, gu, *tensors = ctx.saved_tensors
        p_norm, p_gu, p_down = ctx.refs
        dy = dy.contiguous()
        F_ = w_down.shape[1]
        need1, need2 = p_gu.requires_grad and ctx.meta is not None, p_down.requires_grad
        dy_row, dy_col = MX.quantize(dy, row_tile=MX.A_TILE, col_tile=MX.A_TILE if need2 else None)
        _, w2_col = L.weight_operands(w_down, need_col=True)
        da = MX.gemm(dy_row, w2_col, out_dtype=dy.dtype)
        dw2 = None
        if need2:
            _, a_col = MX.quantize_swiglu(gu, col_tile=MX.b_tile(F_))
            dw2 = _mx_wgrad(p_down, dy_col, a_col)
            del a_col
        dgu_row, dgu_col = MX.quantize_swiglu_bwd(da, gu, row_tile=MX.A_TILE, col_tile=MX.A_TILE if need1 else None)
        del da
        _, w1_col = L.weight_operands(w_gu, need_col=True)
        dxn = MX.gemm(dgu_row, w1_col, out_dtype=dy.dtype)
        dw1 = _mx_wgrad(p_gu, dgu_col, L.Saved.unpack(tensors, ctx.meta)) if need1 else None
        dx, dnw, _ = K.norm_bwd(dxn, h, norm_w, None, mean, rstd, layer_norm=False, dres=dy)
        return dx, _vec_grad(p_norm, dnw), dw1, dw2, None, None


def fused_mlp_eligible(h: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor) -> bool:
    T, D = h.shape
    F2 = w_gu.shape[0]
    return (h.is_cuda and h.dtype == torch.bfloat16 and T % 128 == 0 and D % 128 == 0 and F2 % 256 == 0
            and L.mx_eligible(T, F2, D) and L.mx_eligible(T, D, F2 // 2))


def fused_mlp(h, norm_w, w_gate_up, w_down, eps=1e-5, store_fp8: bool = False):
    """``h + swiglu(rmsnorm(h) W_gu^T) W_down^T`` with MXFP8 GEMMs."""
    return FusedMLPFn.apply(h, norm_w, w_gate_up, w_down, eps, store_fp8)


class SwiGLUFn(Function):
    @staticmethod
    def forward(ctx, gu):
        ctx.save_for_backward(gu)
        return K.swiglu_fwd(gu)

    @staticmethod
    def backward(ctx, da):
        (gu,) = ctx.saved_tensors
        return K.swiglu_bwd(da.contiguous(), gu)


def swiglu(gu):
    return SwiGLUFn.apply(gu)


class GeluFn(Function):
    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        return K.gelu_fwd(x)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return K.gelu_bwd(dy.contiguous(), x)


def gelu(x):
    return GeluFn.apply(x)


class AttentionFn(Function):
    """Rotary embedding + flash attention on a packed ``[T, (Hq + 2 Hkv) * D]`` QKV buffer
    (T = B * S).  The rotation is applied in place to the q and k columns; backward produces the
    packed gradient buffer directly (dk/dv written by the kernel into their columns)."""

    @staticmethod
    def forward(ctx, qkv, sink, cos, sin, B, S, Hq, Hkv, D, causal, window, scale):
        qkv = qkv.contiguous()
        if cos is not None:
            K.rope_(qkv, cos, sin, col0=0, n_heads=Hq + Hkv, head_dim=D, seq_len=S)
        v3 = qkv.view(B, S, -1)
        q = v3[:, :, :Hq * D].unflatten(-1, (Hq, D))
        k = v3[:, :, Hq * D:(Hq + Hkv) * D].unflatten(-1, (Hkv, D))
        v = v3[:, :, (Hq + Hkv) * D:].unflatten(-1, (Hkv, D))
        out, lse = K.attention_fwd(q, k, v, scale=scale, causal=causal, window=window, sink=sink)
        ctx.save_for_backward(qkv, out, lse, sink, cos, sin)
        ctx.cfg = (B, S, Hq, Hkv, D, causal, window, scale)
        return out.view(B * S, Hq * D)

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse, sink, cos, sin = ctx.saved_tensors
        B, S, Hq, Hkv, D, causal, window, scale = ctx.cfg
        v3 = qkv.view(B, S, -1)
        q = v3[:, :, :Hq * D].unflatten(-1, (Hq, D))
        k = v3[:, :, Hq * D:(Hq + Hkv) * D].unflatten(-1, (Hkv, D))
        v = v3[:, :, (Hq + Hkv) * D:].unflatten(-1, (Hkv, D))
        dqkv = torch.empty_like(qkv)
        d3 = dqkv.view(B, S, -1)
        dk = d3[:, :, Hq * D:(Hq + Hkv) * D].unflatten(-1, (Hkv, D))
        dv = d3[:, :, (Hq + Hkv) * D:].unflatten(-1, (Hkv, D))
        dq, _, _, dsink = K.attention_bwd(dout.contiguous().view(B, S, Hq, D), q, k, v, out, lse, scale=scale,
                                          causal=causal, window=window, sink=sink, dk_out=dk, dv_out=dv)
        d3[:, :, :Hq * D].copy_(dq.reshape(B, S, Hq * D))
        if cos is not None:
            K.rope_(dqkv, cos, sin, col0=0, n_heads=Hq + Hkv, head_dim=D, seq_len=S, backward=True)
        if sink is not None and dsink is not None:
            dsink = dsink.to(sink.dtype)
        return dqkv, dsink, None, None, None, None, None, None, None, None, None, None


def attention_packed(qkv, *, B, S, Hq, Hkv, D, cos=None, sin=None, sink=None, causal=True, window=0, scale=None):
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    return AttentionFn.apply(qkv, sink, cos, sin, B, S, Hq, Hkv, D, causal, window, scale)


class RopePackedFn(Function):
    """Rotary embedding of the q and k columns of a packed ``[T, (Hq + 2 Hkv) * D]`` buffer as an
    operator of its own (the context-parallel attention path rotates before the key/value exchange).
    Token ``t`` sits at row ``t % S`` of the tables, so a rank holding a later chunk of the sequence
    passes the matching slice of ``cos`` / ``sin``."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, S, n_heads, D):
        out = qkv.contiguous().clone()
        K.rope_(out, cos, sin, col0=0, n_heads=n_heads, head_dim=D, seq_len=S)
        ctx.save_for_backward(cos, sin)
        ctx.cfg = (S, n_heads, D)
        return out

    @staticmethod
    def backward(ctx, dout):
        cos, sin = ctx.saved_tensors
        S, n_heads, D = ctx.cfg
        d = dout.contiguous().clone()
        K.rope_(d, cos, sin, col0=0, n_heads=n_heads, head_dim=D, seq_len=S, backward=True)
        return d, None, None, None, None, None


def rope_packed(qkv, cos, sin, *, S, Hq, Hkv, D):
    return RopePackedFn.apply(qkv, cos, sin, S, Hq + Hkv, D)


class AttentionBSHDFn(Function):
    """Flash attention on separate ``[B, S, H, D]`` tensors (MMDiT joint attention, tests)."""

    @staticmethod
    def forward(ctx, q, k, v, sink, causal, window, scale):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        out, lse = K.attention_fwd(q, k, v, scale=scale, causal=causal, window=window, sink=sink)
        ctx.save_for_backward(q, k, v, out, lse, sink)
        ctx.cfg = (causal, window, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, sink = ctx.saved_tensors
        causal, window, scale = ctx.cfg
        dq, dk, dv, dsink = K.attention_bwd(dout.contiguous(), q, k, v, out, lse, scale=scale, causal=causal,
                                            window=window, sink=sink)
        return dq.to(q.dtype), dk, dv, (None if dsink is None else dsink.to(sink.dtype)), None, None, None


def attention(q, k, v, *, causal=True, window=0, sink=None, scale=None):
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    return AttentionBSHDFn.apply(q, k, v, sink, causal, window, scale)


class EmbeddingFn(Function):
    @staticmethod
    def forward(ctx, ids, table):
        ctx.save_for_backward(ids)
        ctx.table = table
        return K.gather_rows(table, ids.view(-1))

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        table = ctx.table
        mg = getattr(table, "main_grad", None)
        if mg is not None and mg.dtype == torch.float32:
            K.scatter_add_rows(mg, ids.view(-1), dy.contiguous())
            return None, None
        g = torch.zeros(table.shape, dtype=torch.float32, device=table.device)
        K.scatter_add_rows(g, ids.view(-1), dy.contiguous())
        if mg is not None:
            mg.add_(g.to(mg.dtype))
            return None, None
        return None, g.to(table.dtype)


def embedding(ids, table):
    return EmbeddingFn.apply(ids, table)


class ExpandRowsFn(Function):
    """``out[r] = src[seq[r]]`` for rows grouped by ``seq`` (ascending; group ``b`` = rows ``offsets[b] : offsets[b + 1]``):
    every sample's vector repeated over the sample's tokens.  Backward is the per-group sum of the incoming rows - one
    deterministic segment reduction instead of a sort of ``seq`` and an accumulating index put."""

    @staticmethod
    def forward(ctx, src, seq, offsets):
        ctx.save_for_backward(seq, offsets)
        ctx.shape, ctx.dtype = src.shape, src.dtype
        return K.gather_rows(src, seq.view(-1))

    @staticmethod
    def backward(ctx, g):
        seq, offsets = ctx.saved_tensors
        B, D = ctx.shape
        g = g.contiguous()
        if use_kernels(g) and g.dtype in (torch.bfloat16, torch.float32) and D % 8 == 0:
            from . import _lib
            out = torch.zeros((B, D), dtype=torch.float32, device=g.device)
            seg = offsets.to(torch.int64).contiguous()
            n_seg = torch.full((1,), B, dtype=torch.int64, device=g.device)
            n = g.shape[0]
            partial = torch.empty(int(_lib.load().b200_segment_sum_scratch_elems(n, D)), dtype=torch.float32, device=g.device)
            call("b200_segment_sum_gather", ptr(g), int(g.dtype == torch.float32), n, None, ptr(seg), ptr(n_seg), n, B, D, ptr(out), 0,
                 ptr(partial), stream_ptr())
            return out.to(ctx.dtype), None, None
        out = torch.zeros((B, D), dtype=torch.float32, device=g.device)
        out.index_add_(0, seq.view(-1), g.float())
        return out.to(ctx.dtype), None, None


def expand_rows(src, seq, offsets):
    """``src[seq]`` with a segment-sum backward; ``offsets [B + 1]`` bound the groups of the ascending ``seq``."""
    return ExpandRowsFn.apply(src, seq, offsets)


class LMHeadLossFn(Function):
    """loss = mean CE(norm(x) W^T, labels): final norm, vocabulary GEMM and fused cross-entropy.
    The logits buffer is overwritten with its own gradient during forward, so backward starts
    from dlogits without recomputing the softmax."""

    @staticmethod
    def forward(ctx, x, norm_w, weight, labels, eps, loss_mask_count, precision):
        xn, _, _, rstd = K.norm_fwd(x, norm_w, None, eps)
        keep = L.low_precision(precision, x.shape[0], weight.shape[0], weight.shape[1])
        logits, saved = L.forward(xn, weight, precision, need_wgrad=keep and weight.requires_grad)
        del xn
        n_valid = loss_mask_count if loss_mask_count is not None else max(int(labels.numel()), 1)
        losses = K.cross_entropy_(logits, labels.view(-1), 1.0 / n_valid, write_grad=True)
        tensors, ctx.meta = L.Saved.pack(saved) if saved is not None else ([], None)
        ctx.save_for_backward(x, norm_w, weight, rstd, logits, *tensors)
        ctx.cfg = (eps, precision)
        ctx.refs = (norm_w,)
        return losses.sum() / n_valid

    @staticmethod
    def backward(ctx, dloss):
        x, norm_w, weight, rstd, dlogits, *tensors = ctx.saved_tensors
        eps, precision = ctx.cfg
        if dloss.numel() != 1:
            raise RuntimeError("LMHeadLossFn expects a scalar upstream gradient")
        scale = dloss.reshape(())
        # upstream gradient other than 1 (loss scaling, grad accumulation weights) is applied to dlogits
        dl = dlogits if _is_one(scale) else (dlogits.float() * scale).to(dlogits.dtype)
        if ctx.meta is not None:
            saved = L.Saved.unpack(tensors, ctx.meta)
        elif weight.requires_grad:
            saved = K.norm_fwd(x, norm_w, None, eps)[0]
        else:
            saved = None
        dxn, dw = L.backward(dl, saved, weight, precision, need_dx=True,
                             need_dw=weight.requires_grad and saved is not None)
        del saved
        dx, dnw, _ = K.norm_bwd(dxn, x, norm_w, None, None, rstd)
        return dx, _vec_grad(ctx.refs[0], dnw), dw, None, None, None, None


def _is_one(t: torch.Tensor) -> bool:
    # a host read on CPU only; on CUDA the multiply is always done by the caller's choice below
    if t.is_cuda:
        return getattr(_is_one, "assume_unit", True)
    return float(t) == 1.0


def lm_head_loss(x, norm_w, weight, labels, *, eps=1e-5, n_valid=None, precision="bf16"):
    return LMHeadLossFn.apply(x, norm_w, weight, labels, eps, n_valid, precision)


# --------------------------------------------------------------------------------------
# MMDiT glue: AdaLN modulation, gated residual, rotary embedding on [B, S, H, D]
# --------------------------------------------------------------------------------------
def _mod_ok(x2d, *vecs) -> bool:
    return (use_kernels(x2d) and x2d.dtype == torch.bfloat16 and x2d.shape[1] % 256 == 0 and x2d.shape[1] <= 4096
            and all(v.dtype == torch.bfloat16 and v.stride(-1) == 1 and v.stride(0) % 8 == 0 and v.data_ptr() % 16 == 0 for v in vecs))


class LNModulateFn(Function):
    """``LayerNorm(x) * (1 + scale[b]) + shift[b]`` (no affine; sample ``b`` owns ``S`` consecutive rows):
    one kernel forward, one row kernel + one per-sample column reduction backward."""

    @staticmethod
    def forward(ctx, x, shift, scale, B, eps):
        T, D = x.shape
        S = T // B
        if _mod_ok(x, shift, scale):
            x = x.contiguous()
            y = torch.empty_like(x)
            mean = torch.empty(T, dtype=torch.float32, device=x.device)
            rstd = torch.empty(T, dtype=torch.float32, device=x.device)
            call("b200_ln_modulate_fwd", ptr(x), ptr(shift), ptr(scale), shift.stride(0), ptr(y), ptr(mean), ptr(rstd), T, D, S,
                 float(eps), stream_ptr())
        else:
            xf = x.float()
            mean = xf.mean(-1)
            rstd = torch.rsqrt(xf.var(-1, unbiased=False) + eps)
            xh = (xf - mean[:, None]) * rstd[:, None]
            y = (xh.view(B, S, D) * (1 + scale.float()[:, None]) + shift.float()[:, None]).reshape(T, D).to(x.dtype)
        ctx.save_for_backward(x, scale, mean, rstd)
        ctx.cfg = (B, S, shift.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, scale, mean, rstd = ctx.saved_tensors
        B, S, vdt = ctx.cfg
        T, D = x.shape
        dy = dy.contiguous()
        if _mod_ok(x, scale) and dy.dtype == torch.bfloat16:
            dx = torch.empty_like(x)
            dscale = torch.empty(B, D, dtype=torch.float32, device=x.device)
            dshift = torch.empty(B, D, dtype=torch.float32, device=x.device)
            call("b200_ln_modulate_bwd", ptr(dy), ptr(x), ptr(scale), scale.stride(0), ptr(mean), ptr(rstd), ptr(dx), ptr(dscale),
                 ptr(dshift), T, D, S, stream_ptr())
        else:
            xh = (x.float() - mean[:, None]) * rstd[:, None]
            dyf = dy.float()
            g = (dyf.view(B, S, D) * (1 + scale.float()[:, None])).reshape(T, D)
            dx = (rstd[:, None] * (g - g.mean(-1, keepdim=True) - xh * (g * xh).mean(-1, keepdim=True))).to(x.dtype)
            dscale = (dyf * xh).view(B, S, D).sum(1)
            dshift = dyf.view(B, S, D).sum(1)
        return dx, dshift.to(vdt), dscale.to(vdt), None, None


def ln_modulate(x2d, shift, scale, B, eps=1e-6):
    return LNModulateFn.apply(x2d, shift, scale, B, eps)


class GateResidualFn(Function):
    """``res + y * gate[b]`` with the per-sample gate gradient reduced by a kernel."""

    @staticmethod
    def forward(ctx, res, y, gate, B):
        T, D = y.shape
        S = T // B
        if _mod_ok(y, gate) and res.dtype == torch.bfloat16:
            res, y = res.contiguous(), y.contiguous()
            out = torch.empty_like(y)
            call("b200_gate_residual_fwd", ptr(res), ptr(y), ptr(gate), gate.stride(0), ptr(out), T, D, S, stream_ptr())
        else:
            out = (res.float() + (y.float().view(B, S, D) * gate.float()[:, None]).reshape(T, D)).to(y.dtype)
        ctx.save_for_backward(y, gate)
        ctx.cfg = (B, S)
        return out

    @staticmethod
    def backward(ctx, dout):
        y, gate = ctx.saved_tensors
        B, S = ctx.cfg
        T, D = y.shape
        dout = dout.contiguous()
        if _mod_ok(y, gate) and dout.dtype == torch.bfloat16:
            dy = torch.empty_like(y)
            dgate = torch.empty(B, D, dtype=torch.float32, device=y.device)
            call("b200_gate_residual_bwd", ptr(dout), ptr(y), ptr(gate), gate.stride(0), ptr(dy), ptr(dgate), T, D, S, stream_ptr())
        else:
            df = dout.float()
            dy = (df.view(B, S, D) * gate.float()[:, None]).reshape(T, D).to(y.dtype)
            dgate = (df * y.float()).view(B, S, D).sum(1)
        return dout, dy, dgate.to(gate.dtype), None


def gate_residual(res2d, y2d, gate, B):
    return GateResidualFn.apply(res2d, y2d, gate, B)


class RopeBSHDFn(Function):
    """Rotate-half rotary embedding of ``x [B, S, H, D]`` with tables ``[S, D / 2]`` (1-D or n-D positions:
    the tables carry them); backward is the inverse rotation of the gradient."""

    @staticmethod
    def forward(ctx, x, cos, sin):
        B, S, H, D = x.shape
        out = x.contiguous().clone()
        K.rope_(out.view(B * S, H * D), cos, sin, col0=0, n_heads=H, head_dim=D, seq_len=S)
        ctx.save_for_backward(cos, sin)
        return out

    @staticmethod
    def backward(ctx, g):
        cos, sin = ctx.saved_tensors
        B, S, H, D = g.shape
        g = g.contiguous().clone()
        K.rope_(g.view(B * S, H * D), cos, sin, col0=0, n_heads=H, head_dim=D, seq_len=S, backward=True)
        return g, None, None


def rope_bshd(x, cos, sin):
    return RopeBSHDFn.apply(x, cos, sin)


# --------------------------------------------------------------------------------------
# MoE router projection
# --------------------------------------------------------------------------------------
class RouterLogitsFn(Function):
    """fp32 router logits ``hn W^T`` with ``W [E, d]`` kept in fp32, on the bf16 tensor-core GEMM: the
    weight is split into a bf16 head and a bf16 remainder (``W = hi + lo`` to ~16 mantissa bits) and the
    two products accumulate in fp32, so the logits match an fp32-weight GEMM of the bf16 activations to
    rounding; the backward GEMMs take the logit gradient in bf16 (the reference's Megatron patch runs the
    router backward in bf16 as well: small_llm_moe_pretraining/primus/patches)."""

    @staticmethod
    def forward(ctx, hn, router):
        ctx.save_for_backward(hn, router)
        if not use_kernels(hn) or hn.dtype != torch.bfloat16 or hn.shape[1] % 8 or router.shape[0] % 8:
            return hn.float() @ router.float().t()
        hi = router.detach().to(torch.bfloat16)
        lo = (router.detach().float() - hi.float()).to(torch.bfloat16)
        out = K.gemm(hn.contiguous(), hi, out_dtype=torch.float32)
        K.gemm(hn.contiguous(), lo, out=out, accumulate=True)
        return out

    @staticmethod
    def backward(ctx, dl):
        hn, router = ctx.saved_tensors
        if not use_kernels(hn) or hn.dtype != torch.bfloat16 or hn.shape[1] % 8 or router.shape[0] % 8:
            return (dl.float() @ router.float()).to(hn.dtype), (dl.float().t() @ hn.float()).to(router.dtype)
        g = dl.to(torch.bfloat16).contiguous()
        dhn = K.gemm(g, router.detach().to(torch.bfloat16).contiguous(), b_mn_major=True) if ctx.needs_input_grad[0] else None
        dw = K.gemm(g, hn.contiguous(), a_mn_major=True, b_mn_major=True, out_dtype=torch.float32).to(router.dtype) \
            if ctx.needs_input_grad[1] else None
        return dhn, dw


def router_logits(hn, router):
    return RouterLogitsFn.apply(hn, router)
