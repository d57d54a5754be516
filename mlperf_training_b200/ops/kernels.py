"""Raw (non-autograd) operators.  Each function has two bodies with identical semantics:

* CUDA tensors  -> the hand-written sm_100a kernel through ``_lib.call`` (loud failure if the
  library is missing);
* CPU tensors   -> the eager PyTorch definition, which is also the oracle the GPU tests
  compare against (the role ``generative_recommenders/ops/pytorch/*`` plays in the
  reference, selected there by ``HammerKernel.PYTORCH``, generative_recommenders/common.py:115-125).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import _lib
from ._lib import call, ptr, stream_ptr, use_kernels

BF16 = torch.bfloat16


def _row_major(t: torch.Tensor) -> torch.Tensor:
    """2-D tensor with unit inner stride, 16-byte aligned base and pitch."""
    if t.dim() != 2:
        raise ValueError(f"expected a 2-D tensor, got shape {tuple(t.shape)}")
    esz = t.element_size()
    if t.stride(1) != 1 or (t.stride(0) * esz) % 16 != 0 or t.data_ptr() % 16 != 0 or t.stride(0) < t.shape[1]:
        per16 = 16 // esz
        cols = (t.shape[1] + per16 - 1) // per16 * per16
        if cols == t.shape[1]:
            t = t.contiguous()
        else:  # TMA needs a 16-byte row pitch: copy into a padded buffer and view the valid columns
            buf = torch.zeros((t.shape[0], cols), dtype=t.dtype, device=t.device)
            buf[:, :t.shape[1]].copy_(t)
            t = buf[:, :t.shape[1]]
    return t


# --------------------------------------------------------------------------------------
# GEMM
# --------------------------------------------------------------------------------------
def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn_major: bool = False, b_mn_major: bool = False,
         out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None, accumulate: bool = False,
         bias: torch.Tensor | None = None, residual: torch.Tensor | None = None,
         alpha: float = 1.0) -> torch.Tensor:
    """``D[M,N] (+)= alpha * A @ B^T (+ bias[N]) (+ residual[M,N])`` with bf16 operands.

    ``a`` is ``[M,K]`` (K-major) or, with ``a_mn_major``, ``[K,M]``; ``b`` is ``[N,K]`` or, with
    ``b_mn_major``, ``[K,N]``.  So ``gemm(x, w)`` is ``x @ w.T`` (forward),
    ``gemm(dy, w, b_mn_major=True)`` is ``dy @ w`` (dgrad) and
    ``gemm(dy, x, a_mn_major=True, b_mn_major=True)`` is ``dy.T @ x`` (wgrad).
    """
    M, K = (a.shape[1], a.shape[0]) if a_mn_major else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn_major else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"gemm: contraction mismatch {K} vs {Kb}")
    if out is not None:
        out_dtype = out.dtype
    elif out_dtype is None:
        out_dtype = a.dtype
    if not use_kernels(a):
        am = a.float().t() if a_mn_major else a.float()
        bm = b.float() if b_mn_major else b.float().t()
        d = alpha * (am @ bm)
        if bias is not None:
            d = d + bias.float()
        if residual is not None:
            d = d + residual.float()
        if out is None:
            return d.to(out_dtype)
        if accumulate:
            out.add_(d.to(out.dtype))
        else:
            out.copy_(d.to(out.dtype))
        return out
    if a.dtype != BF16 or b.dtype != BF16:
        raise TypeError("gemm: operands must be bf16")
    a = _row_major(a)
    b = _row_major(b)
    if out is None:
        if accumulate:
            raise ValueError("gemm: accumulate needs an output tensor")
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    elif out.dim() != 2 or out.shape[0] != M or out.shape[1] != N or out.stride(1) != 1:
        raise ValueError(f"gemm: bad output {tuple(out.shape)} for {M}x{N}")
    if out.dtype not in (BF16, torch.float32):
        raise TypeError("gemm: output must be bf16 or fp32")
    if (out.stride(0) * out.element_size()) % 16 != 0 or out.data_ptr() % 16 != 0:
        raise ValueError("gemm: output pitch/base must be 16-byte aligned")
    if bias is not None:
        bias = bias.to(BF16).contiguous()
    ldr = 0
    if residual is not None:
        if residual.dtype != BF16 or residual.stride(1) != 1:
            residual = residual.to(BF16).contiguous()
        ldr = residual.stride(0)
    call("b200_gemm_bf16", ptr(a), ptr(b), ptr(out), M, N, K, a.stride(0), b.stride(0), out.stride(0),
         int(a_mn_major), int(b_mn_major), int(out.dtype == torch.float32), int(accumulate), ptr(bias),
         ptr(residual), ldr, float(alpha), stream_ptr())
    return out


# --------------------------------------------------------------------------------------
# normalisation
# --------------------------------------------------------------------------------------
def norm_fwd(x: torch.Tensor, weight: torch.Tensor | None, bias: torch.Tensor | None, eps: float, *,
             layer_norm: bool = False, swish: bool = False, residual: torch.Tensor | None = None):
    """Returns ``(y, h, mean, rstd)``.  ``h = x + residual`` (or ``x``) is what was normalised;
    RMSNorm when ``layer_norm`` is False; ``swish`` gives ``h * sigmoid(norm(h))``."""
    T, D = x.shape
    if not use_kernels(x):
        h = x.float() if residual is None else (x.float() + residual.float()).to(x.dtype).float()
        if layer_norm:
            mean = h.mean(-1)
            var = ((h - mean[:, None]) ** 2).mean(-1)
            rstd = torch.rsqrt(var + eps)
            n = (h - mean[:, None]) * rstd[:, None]
        else:
            mean = None
            rstd = torch.rsqrt((h * h).mean(-1) + eps)
            n = h * rstd[:, None]
        if weight is not None:
            n = n * weight.float()
        if bias is not None:
            n = n + bias.float()
        y = h * torch.sigmoid(n) if swish else n
        return y.to(x.dtype), h.to(x.dtype), mean, rstd
    x = x.contiguous()
    y = torch.empty_like(x)
    h = x
    if residual is not None:
        residual = residual.contiguous()
        h = torch.empty_like(x)
    mean = torch.empty(T, dtype=torch.float32, device=x.device) if layer_norm else None
    rstd = torch.empty(T, dtype=torch.float32, device=x.device)
    w = None if weight is None else weight.to(BF16).contiguous()
    b = None if bias is None else bias.to(BF16).contiguous()
    call("b200_norm_fwd", int(layer_norm), ptr(x), ptr(residual), ptr(w), ptr(b), ptr(y),
         ptr(h) if residual is not None else None, ptr(mean), ptr(rstd), T, D, float(eps), int(swish), stream_ptr())
    return y, h, mean, rstd


def norm_bwd(dy: torch.Tensor, h: torch.Tensor, weight: torch.Tensor | None, bias: torch.Tensor | None,
             mean: torch.Tensor | None, rstd: torch.Tensor, *, layer_norm: bool = False, swish: bool = False,
             dres: torch.Tensor | None = None, dw_out: torch.Tensor | None = None,
             db_out: torch.Tensor | None = None, accumulate: bool = False):
    """Returns ``(dx, dw, db)`` (dw/db fp32).  ``dres`` is added to ``dx`` (gradient arriving on
    the residual branch).  With ``dw_out``/``db_out`` the gradients are written (or added when
    ``accumulate``) in place."""
    T, D = h.shape
    if not use_kernels(h):
        hf, dyf = h.float(), dy.float()
        mu = mean[:, None] if layer_norm else 0.0
        xn = (hf - mu) * rstd[:, None]
        w = weight.float() if weight is not None else torch.ones(D)
        if swish:
            n = xn * w + (bias.float() if bias is not None else 0.0)
            s = torch.sigmoid(n)
            dn = dyf * hf * s * (1 - s)
            direct = dyf * s
        else:
            dn = dyf
            direct = 0.0
        dw = (dn * xn).sum(0)
        db = dn.sum(0)
        g = dn * w
        s1 = (g * xn).mean(-1, keepdim=True)
        s2 = g.mean(-1, keepdim=True) if layer_norm else 0.0
        dx = rstd[:, None] * (g - xn * s1 - s2) + direct
        if dres is not None:
            dx = dx + dres.float()
        if dw_out is not None:
            dw_out.copy_(dw_out + dw if accumulate else dw)
            dw = dw_out
        if db_out is not None:
            db_out.copy_(db_out + db if accumulate else db)
            db = db_out
        return dx.to(h.dtype), dw, db
    dy = dy.contiguous()
    h = h.contiguous()
    dx = torch.empty_like(h)
    w = None if weight is None else weight.to(BF16).contiguous()
    b = None if bias is None else bias.to(BF16).contiguous()
    want_w = weight is not None
    want_b = bias is not None
    dw = dw_out if dw_out is not None else (torch.empty(D, dtype=torch.float32, device=h.device) if want_w else None)
    db = db_out if db_out is not None else (torch.empty(D, dtype=torch.float32, device=h.device) if want_b else None)
    lib = _lib.load()
    scratch = None
    if want_w or want_b:
        n = lib.b200_norm_bwd_scratch_elems(T, D)
        scratch = torch.empty(n, dtype=torch.float32, device=h.device)
    if dres is not None:
        dres = dres.contiguous()
    call("b200_norm_bwd", int(layer_norm), ptr(dy), ptr(h), ptr(w), ptr(b), ptr(mean), ptr(rstd), ptr(dres), ptr(dx),
         ptr(dw), ptr(db), ptr(scratch), T, D, int(swish), int(accumulate), stream_ptr())
    return dx, dw, db


# --------------------------------------------------------------------------------------
# rotary embedding
# --------------------------------------------------------------------------------------
def rope_tables(seq_len: int, head_dim: int, theta: float, device, scaling: float = 1.0):
    """fp32 cos/sin tables ``[seq_len, head_dim/2]`` for the rotate-half convention."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    pos = torch.arange(seq_len, dtype=torch.float64) / scaling
    ang = torch.outer(pos, inv)
    return ang.cos().float().to(device), ang.sin().float().to(device)


def rope_(buf: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, *, col0: int, n_heads: int, head_dim: int,
          seq_len: int, positions: torch.Tensor | None = None, backward: bool = False) -> torch.Tensor:
    """In-place rotation of ``n_heads`` heads stored at columns ``col0 ..`` of the rows of
    ``buf`` ``[T, row]``.  Token ``t`` sits at position ``positions[t]`` or ``t % seq_len``."""
    T = buf.shape[0]
    if not use_kernels(buf):
        half = head_dim // 2
        pos = positions.long() if positions is not None else torch.arange(T, device=buf.device) % seq_len
        c = cos[pos][:, None, :]
        s = sin[pos][:, None, :] * (-1.0 if backward else 1.0)
        view = buf[:, col0:col0 + n_heads * head_dim].reshape(T, n_heads, head_dim).float()
        x1, x2 = view[..., :half], view[..., half:]
        out = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
        buf[:, col0:col0 + n_heads * head_dim] = out.reshape(T, n_heads * head_dim).to(buf.dtype)
        return buf
    if buf.stride(1) != 1:
        raise ValueError("rope_: rows must be contiguous")
    pos32 = None if positions is None else positions.to(torch.int32).contiguous()
    call("b200_rope", ptr(buf), ptr(cos), ptr(sin), ptr(pos32), T, seq_len, buf.stride(0), col0, n_heads, head_dim,
         int(backward), stream_ptr())
    return buf


# --------------------------------------------------------------------------------------
# activations
# --------------------------------------------------------------------------------------
def swiglu_fwd(gu: torch.Tensor) -> torch.Tensor:
    T, F2 = gu.shape
    Fh = F2 // 2
    if not use_kernels(gu):
        g, u = gu[:, :Fh].float(), gu[:, Fh:].float()
        return (F.silu(g) * u).to(gu.dtype)
    gu = gu.contiguous()
    out = torch.empty((T, Fh), dtype=gu.dtype, device=gu.device)
    call("b200_swiglu_fwd", ptr(gu), ptr(out), T, Fh, stream_ptr())
    return out


def swiglu_bwd(da: torch.Tensor, gu: torch.Tensor) -> torch.Tensor:
    T, F2 = gu.shape
    Fh = F2 // 2
    if not use_kernels(gu):
        g, u, d = gu[:, :Fh].float(), gu[:, Fh:].float(), da.float()
        s = torch.sigmoid(g)
        dg = d * u * s * (1 + g * (1 - s))
        du = d * g * s
        return torch.cat([dg, du], dim=1).to(gu.dtype)
    gu = gu.contiguous()
    da = da.contiguous()
    out = torch.empty_like(gu)
    call("b200_swiglu_bwd", ptr(da), ptr(gu), ptr(out), T, Fh, stream_ptr())
    return out


def gelu_fwd(x: torch.Tensor) -> torch.Tensor:
    if not use_kernels(x):
        return F.gelu(x.float(), approximate="tanh").to(x.dtype)
    x = x.contiguous()
    y = torch.empty_like(x)
    call("b200_gelu_fwd", ptr(x), ptr(y), x.numel(), stream_ptr())
    return y


def gelu_bwd(dy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    if not use_kernels(x):
        xf = x.float().detach().requires_grad_(True)
        with torch.enable_grad():
            y = F.gelu(xf, approximate="tanh")
        (g,) = torch.autograd.grad(y, xf, dy.float())
        return g.to(x.dtype)
    x = x.contiguous()
    dy = dy.contiguous()
    dx = torch.empty_like(x)
    call("b200_gelu_bwd", ptr(dy), ptr(x), ptr(dx), x.numel(), stream_ptr())
    return dx


# --------------------------------------------------------------------------------------
# embedding rows
# --------------------------------------------------------------------------------------
def gather_rows(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    if not use_kernels(table):
        # ids outside [0, rows) give zero rows, as in the kernel
        out = table[ids.clamp(min=0, max=table.shape[0] - 1)]
        return torch.where(((ids >= 0) & (ids < table.shape[0]))[:, None], out, torch.zeros_like(out))
    ids = ids.to(torch.int64).contiguous()
    table = table.contiguous()
    out = torch.empty((ids.numel(), table.shape[1]), dtype=table.dtype, device=table.device)
    call("b200_gather_rows", ptr(table), ptr(ids), ptr(out), ids.numel(), table.shape[1], table.shape[0], stream_ptr())
    return out


def scatter_add_rows(grad: torch.Tensor, ids: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    """``grad[ids[t]] += dy[t]`` with fp32 ``grad`` and bf16 ``dy``."""
    if not use_kernels(grad):
        ok = ids >= 0
        grad.index_add_(0, ids[ok], dy[ok].to(grad.dtype))
        return grad
    ids = ids.to(torch.int64).contiguous()
    dy = dy.contiguous()
    call("b200_scatter_add_rows", ptr(dy), ptr(ids), ptr(grad), ids.numel(), grad.shape[1], grad.shape[0], stream_ptr())
    return grad


def accum_f32_(acc: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """``acc (fp32) += src (bf16)``."""
    if not use_kernels(acc) or acc.numel() % 8 != 0:
        acc.add_(src.to(acc.dtype))
        return acc
    call("b200_accum_f32_bf16", ptr(acc), ptr(src.contiguous()), acc.numel(), stream_ptr())
    return acc


# --------------------------------------------------------------------------------------
# cross-entropy
# --------------------------------------------------------------------------------------
def cross_entropy_(logits: torch.Tensor, labels: torch.Tensor, grad_scale: float, *, write_grad: bool = True,
                   ignore_index: int = -100):
    """Per-token loss (fp32) of bf16 ``logits`` ``[T,V]``; when ``write_grad`` the logits are
    overwritten with ``(softmax - onehot) * grad_scale`` (zero rows for ignored labels)."""
    T, V = logits.shape
    if not use_kernels(logits):
        lf = logits.float()
        lse = torch.logsumexp(lf, dim=-1)
        valid = (labels != ignore_index)
        safe = labels.clamp(min=0)
        loss = torch.where(valid, lse - lf.gather(1, safe[:, None])[:, 0], torch.zeros_like(lse))
        if write_grad:
            p = torch.softmax(lf, dim=-1)
            p[torch.arange(T), safe] -= 1.0
            p = p * grad_scale * valid[:, None]
            logits.copy_(p.to(logits.dtype))
        return loss
    if logits.stride(1) != 1:
        raise ValueError("cross_entropy_: logits rows must be contiguous")
    labels = labels.to(torch.int64).contiguous()
    loss = torch.empty(T, dtype=torch.float32, device=logits.device)
    call("b200_cross_entropy", ptr(logits), ptr(labels), ptr(loss), None, T, logits.stride(0), V, float(grad_scale),
         int(write_grad), int(ignore_index), stream_ptr())
    return loss


# --------------------------------------------------------------------------------------
# optimizer
# --------------------------------------------------------------------------------------
def sumsq(g: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    """``out[0] (+)= sum(g^2)`` in fp32 with a fixed reduction order."""
    if not use_kernels(g):
        s = (g.float() ** 2).sum()
        out[0] = out[0] + s if accumulate else s
        return out
    g = g.contiguous().view(-1)
    n_scr = _lib.load().b200_sumsq_scratch_elems()
    scratch = torch.empty(n_scr, dtype=torch.float32, device=g.device)
    call("b200_sumsq", ptr(g), g.numel(), int(g.dtype == BF16), ptr(scratch), ptr(out), int(accumulate), stream_ptr())
    return out


def adamw_(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, *, lr: float, beta1: float,
           beta2: float, eps: float, weight_decay: float, step: int, master: torch.Tensor | None = None,
           grad_scale: float = 1.0, sumsq_buf: torch.Tensor | None = None, max_norm: float = 0.0,
           zero_grad: bool = False) -> None:
    """Fused AdamW on flat buffers.  ``sumsq_buf`` (device scalar holding the squared global
    gradient norm, before ``grad_scale``) with ``max_norm > 0`` folds gradient clipping in.
    ``m`` and ``v`` are both fp32 or both bf16; with bf16 the update is computed in fp32 from the stored
    values and the new moments are rounded to nearest on the way back."""
    if m.dtype != v.dtype or m.dtype not in (torch.float32, BF16):
        raise ValueError("adamw_: moments must both be fp32 or both be bf16")
    if not use_kernels(p):
        gf = g.float() * grad_scale
        if sumsq_buf is not None and max_norm > 0:
            norm = sumsq_buf[0].sqrt() * grad_scale
            coef = max_norm / (norm + 1e-6)
            if coef < 1:
                gf = gf * coef
        w = master if master is not None else p.float()
        mf = m.float().mul_(beta1).add_(gf, alpha=1 - beta1)
        vf = v.float().mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
        m.copy_(mf)
        v.copy_(vf)
        mhat = mf / (1 - beta1 ** step)
        vhat = vf / (1 - beta2 ** step)
        w = w * (1 - lr * weight_decay) - lr * mhat / (vhat.sqrt() + eps)
        if master is not None:
            master.copy_(w)
        p.copy_(w.to(p.dtype))
        if zero_grad:
            g.zero_()
        return
    for t in (p, g, m, v):
        if not t.is_contiguous():
            raise ValueError("adamw_: flat contiguous buffers required")
    call("b200_adamw_bf16m" if m.dtype == BF16 else "b200_adamw", ptr(p), int(p.dtype == BF16), ptr(master), ptr(g), int(g.dtype == BF16), ptr(m), ptr(v),
         p.numel(), float(lr), float(beta1), float(beta2), float(eps), float(weight_decay), int(step),
         float(grad_scale), ptr(sumsq_buf), float(max_norm), int(zero_grad), stream_ptr())


# --------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------
def _attn_mask(Sq: int, Skv: int, causal: bool, window: int, device) -> torch.Tensor:
    qp = torch.arange(Sq, device=device)[:, None] + (Skv - Sq)
    kp = torch.arange(Skv, device=device)[None, :]
    ok = torch.ones(Sq, Skv, dtype=torch.bool, device=device)
    if causal:
        ok &= kp <= qp
    if window > 0:
        ok &= (qp - kp) < window
    return ok


def attention_reference(q, k, v, *, scale: float, causal: bool, window: int = 0, sink=None):
    """fp32 eager attention on ``[B,S,H,D]`` tensors; returns ``(out, lse)``.  With ``sink``
    ([Hq] logits) the softmax has one extra column per head that carries no value."""
    B, Sq, Hq, D = q.shape
    Skv, Hkv = k.shape[1], k.shape[2]
    g = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    ok = _attn_mask(Sq, Skv, causal, window, q.device)
    s = s.masked_fill(~ok, float("-inf"))
    if sink is not None:
        sk = sink.float().view(1, Hq, 1, 1).expand(B, Hq, Sq, 1)
        full = torch.cat([s, sk], dim=-1)
        lse = torch.logsumexp(full, dim=-1)
    else:
        lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])
    o = torch.matmul(p, vf).permute(0, 2, 1, 3)
    return o, lse


def attention_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float | None = None,
                  causal: bool = True, window: int = 0, sink: torch.Tensor | None = None):
    """``q`` ``[B,Sq,Hq,D]``, ``k``/``v`` ``[B,Skv,Hkv,D]`` (views into a packed QKV buffer are
    fine: only the head dim must be contiguous).  Returns ``(out [B,Sq,Hq,D], lse [B,Hq,Sq])``."""
    B, Sq, Hq, D = q.shape
    Skv, Hkv = k.shape[1], k.shape[2]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if not use_kernels(q):
        o, lse = attention_reference(q, k, v, scale=scale, causal=causal, window=window, sink=sink)
        return o.to(q.dtype).contiguous(), lse
    for t in (q, k, v):
        if t.stride(3) != 1 or t.stride(2) != D:
            raise ValueError("attention_fwd: heads must be contiguous inside a token row")
    out = torch.empty((B, Sq, Hq, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
    sk = None if sink is None else sink.float().contiguous()
    call("b200_attn_fwd", ptr(q), ptr(k), ptr(v), ptr(out), ptr(lse), ptr(sk), B, Sq, Skv, Hq, Hkv, D,
         q.stride(1), k.stride(1), v.stride(1), out.stride(1), q.stride(0), k.stride(0), v.stride(0), out.stride(0),
         float(scale), int(causal), int(window), stream_ptr())
    return out, lse


def attention_bwd(dout, q, k, v, out, lse, *, scale: float | None = None, causal: bool = True, window: int = 0,
                  sink: torch.Tensor | None = None, dk_out=None, dv_out=None):
    """Returns ``(dq fp32 [B,Sq,Hq,D], dk, dv, dsink)``; ``dk_out``/``dv_out`` may be views into
    a packed gradient buffer."""
    B, Sq, Hq, D = q.shape
    Skv, Hkv = k.shape[1], k.shape[2]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if not use_kernels(q):
        qf = q.float().detach().requires_grad_(True)
        kf = k.float().detach().requires_grad_(True)
        vf = v.float().detach().requires_grad_(True)
        sf = None if sink is None else sink.float().detach().requires_grad_(True)
        with torch.enable_grad():
            o, _ = attention_reference(qf, kf, vf, scale=scale, causal=causal, window=window, sink=sf)
        ins = [qf, kf, vf] + ([sf] if sf is not None else [])
        grads = torch.autograd.grad(o, ins, dout.float())
        dq, dk, dv = grads[0], grads[1].to(k.dtype), grads[2].to(v.dtype)
        if dk_out is not None:
            dk_out.copy_(dk)
            dk = dk_out
        if dv_out is not None:
            dv_out.copy_(dv)
            dv = dv_out
        return dq, dk, dv, (grads[3] if sf is not None else None)
    dout = dout if (dout.stride(3) == 1 and dout.stride(2) == D) else dout.contiguous()
    delta = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
    call("b200_attn_delta", ptr(out), ptr(dout), ptr(delta), B, Sq, Hq, D, out.stride(1), dout.stride(1),
         out.stride(0), dout.stride(0), stream_ptr())
    dq = torch.zeros((B, Sq, Hq, D), dtype=torch.float32, device=q.device)
    dk = dk_out if dk_out is not None else torch.empty((B, Skv, Hkv, D), dtype=k.dtype, device=k.device)
    dv = dv_out if dv_out is not None else torch.empty((B, Skv, Hkv, D), dtype=v.dtype, device=v.device)
    call("b200_attn_bwd", ptr(q), ptr(k), ptr(v), ptr(dout), ptr(lse), ptr(delta), ptr(dq), ptr(dk), ptr(dv), B, Sq,
         Skv, Hq, Hkv, D, q.stride(1), k.stride(1), v.stride(1), dout.stride(1), dk.stride(1), dv.stride(1),
         q.stride(0), k.stride(0), v.stride(0), dout.stride(0), dk.stride(0), dv.stride(0), float(scale),
         int(causal), int(window), stream_ptr())
    dsink = None
    if sink is not None:
        # d/dsink of the extra softmax column: -sum_rows exp(sink - lse) * delta
        dsink = -(torch.exp(sink.float().view(1, Hq, 1) - lse) * delta).sum(dim=(0, 2))
    return dq, dk, dv, dsink
