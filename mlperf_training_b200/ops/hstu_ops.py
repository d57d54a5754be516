"""HSTU operators: jagged pointwise-SiLU attention (forward / backward) and its eager oracle.

``hstu_attention(q, k, v, offsets, max_len, alpha, num_targets, contextual)`` works on jagged
``[L, H, D]`` tensors (views into the fused ``uvqk`` projection buffer are fine: only the head dim
must be contiguous).  Math and mask follow the reference oracle
(generative_recommenders/ops/pytorch/pt_hstu_attention.py:33-84 mask, :130-187 attention):
``O = (silu(alpha Q K^T) / N * mask) V`` with N the static maximum sequence length.
"""
from __future__ import annotations

import torch
from torch.autograd import Function

from . import _lib
from ._lib import call, ptr, stream_ptr, use_kernels


def valid_mask(length: int, n_targets: int = 0, contextual: int = 0, device="cpu") -> torch.Tensor:
    """Boolean ``[len, len]`` visibility matrix of one sequence (rows = queries)."""
    pos = torch.arange(length, device=device)
    max_id = length - n_targets - max(contextual - 1, 0)
    ids = (pos - contextual + (1 if contextual > 0 else 0)).clamp(min=0, max=max_id)
    row, col = ids[:, None], ids[None, :]
    vis = (pos[:, None] == pos[None, :]) | (row > col)
    if contextual > 0:
        vis = vis | ((row == 0) & (pos[None, :] < length - n_targets))
    return vis


def hstu_attention_reference(q, k, v, offsets, max_len: int, alpha: float, num_targets=None, contextual: int = 0):
    """fp32 eager oracle on jagged inputs; returns ``[L, H, D]`` fp32."""
    out = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    offs = offsets.tolist()
    for b in range(len(offs) - 1):
        lo, hi = offs[b], offs[b + 1]
        if hi <= lo:
            continue
        nt = int(num_targets[b]) if num_targets is not None else 0
        qb, kb, vb = (t[lo:hi].float().transpose(0, 1) for t in (q, k, v))     # [H, len, D]
        s = torch.matmul(qb, kb.transpose(-1, -2)) * alpha
        p = torch.nn.functional.silu(s) / max_len
        p = p * valid_mask(hi - lo, nt, contextual, q.device)[None]
        out[lo:hi] = torch.matmul(p, vb).transpose(0, 1)
    return out


def hstu_attention_fp8_reference(q, k, v, offsets, max_len: int, alpha: float, num_targets=None, contextual: int = 0,
                                 scales=None):
    """Eager emulation of the 8-bit forward: Q, K, V rounded to per-tensor e4m3, the activation ``silu(alpha s)``
    rounded to e4m3 before it meets V, ``1 / N`` applied to the output.  ``scales``: the three ``DelayedScale`` states
    (None: every tensor's own maximum)."""
    from . import fp8 as F8
    deq = []
    for i, t in enumerate((q, k, v)):
        if scales is not None:
            sc = scales[i].scale.to(t.device).float()
        else:
            sc = F8.FMAX["e4m3"] / t.detach().abs().amax().float().clamp_min(1e-30)
        deq.append((t.float() * sc).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float() / sc)
    qd, kd, vd = deq
    out = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    offs = offsets.tolist()
    for b in range(len(offs) - 1):
        lo, hi = offs[b], offs[b + 1]
        if hi <= lo:
            continue
        nt = int(num_targets[b]) if num_targets is not None else 0
        qb, kb, vb = (t[lo:hi].transpose(0, 1) for t in (qd, kd, vd))
        s = torch.matmul(qb, kb.transpose(-1, -2)) * alpha
        p = torch.nn.functional.silu(s) * valid_mask(hi - lo, nt, contextual, q.device)[None]
        p = p.clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float()
        out[lo:hi] = (torch.matmul(p, vb) / max_len).transpose(0, 1)
    return out


def _fp8_sites(owner, device):
    """Delayed-scaling states of Q, K, V for the module (or any object) that owns this attention call."""
    from . import fp8 as F8
    sites = getattr(owner, "_attn_fp8_sites", None) if owner is not None else None
    if sites is None:
        sites = tuple(F8.DelayedScale("e4m3", device) for _ in range(3))
        if owner is not None:
            owner._attn_fp8_sites = sites
    return sites


class HstuAttentionFn(Function):
    @staticmethod
    def forward(ctx, q, k, v, offsets, max_len, alpha, num_targets, contextual, fp8_owner=False):
        ctx.cfg = (max_len, alpha, contextual)
        use_fp8 = fp8_owner is not False and q.shape[2] == 128
        if not use_kernels(q):
            ctx.save_for_backward(q, k, v, offsets, num_targets)
            if use_fp8:
                return hstu_attention_fp8_reference(q, k, v, offsets, max_len, alpha, num_targets, contextual).to(q.dtype)
            return hstu_attention_reference(q, k, v, offsets, max_len, alpha, num_targets, contextual).to(q.dtype)
        L, H, D = q.shape
        for t in (q, k, v):
            if t.stride(2) != 1 or t.stride(1) != D:
                raise ValueError("hstu_attention: heads must be contiguous inside a row")
        offs = offsets.to(torch.int32).contiguous()
        nt = None if num_targets is None else num_targets.to(torch.int32).contiguous()
        out = torch.zeros((L, H, D), dtype=q.dtype, device=q.device)
        if use_fp8 and q.dtype == torch.bfloat16:
            # e4m3 forward (delayed per-tensor factors); the backward below runs on the bf16 tensors
            from . import fp8 as F8
            from .linear import weight_epoch
            ops = []
            for t, st in zip((q, k, v), _fp8_sites(fp8_owner, q.device)):
                t2 = t.as_strided((L, H * D), (t.stride(0), 1))      # heads are contiguous inside a row
                st.prepare(t2, weight_epoch())
                ops.append(F8.quantize_rows(t2, st))
            call("b200_hstu_attn_fwd_fp8", ptr(ops[0].q), ptr(ops[1].q), ptr(ops[2].q), ptr(out), ptr(offs), ptr(nt),
                 offs.numel() - 1, L, H, D, int(max_len), int(contextual), H * D, H * D, H * D, out.stride(0), float(alpha),
                 ptr(ops[0].inv_scale), ptr(ops[1].inv_scale), ptr(ops[2].inv_scale), stream_ptr())
        else:
            call("b200_hstu_attn_fwd", ptr(q), ptr(k), ptr(v), ptr(out), ptr(offs), ptr(nt), offs.numel() - 1, L, H, D,
                 int(max_len), int(contextual), q.stride(0), k.stride(0), v.stride(0), out.stride(0), float(alpha),
                 stream_ptr())
        ctx.save_for_backward(q, k, v, offs, nt)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, offs, nt = ctx.saved_tensors
        max_len, alpha, contextual = ctx.cfg
        if not use_kernels(q):
            qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
            with torch.enable_grad():
                o = hstu_attention_reference(qf, kf, vf, offs, max_len, alpha, nt, contextual)
            dq, dk, dv = torch.autograd.grad(o, (qf, kf, vf), dout.float())
            return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None, None, None, None, None, None
        L, H, D = q.shape
        dout = dout if (dout.stride(2) == 1 and dout.stride(1) == D) else dout.contiguous()
        dq = torch.zeros((L, H, D), dtype=torch.float32, device=q.device)
        dk = torch.zeros((L, H, D), dtype=k.dtype, device=q.device)
        dv = torch.zeros((L, H, D), dtype=v.dtype, device=q.device)
        call("b200_hstu_attn_bwd", ptr(q), ptr(k), ptr(v), ptr(dout), ptr(dq), ptr(dk), ptr(dv), ptr(offs), ptr(nt),
             offs.numel() - 1, L, H, D, int(max_len), int(contextual), q.stride(0), k.stride(0), v.stride(0),
             dout.stride(0), dk.stride(0), dv.stride(0), float(alpha), stream_ptr())
        return dq.to(q.dtype), dk, dv, None, None, None, None, None, None


def hstu_attention(q, k, v, offsets, max_len: int, alpha: float, num_targets=None, contextual: int = 0,
                   precision: str = "bf16", owner=None):
    """``precision="fp8"`` (head dim 128): the forward runs on per-tensor e4m3 copies of Q, K, V whose delayed-scaling
    states live on ``owner`` (the calling module; None = fresh states, i.e. every call uses its own maxima); the
    backward uses the bf16 tensors."""
    fp8_owner = (owner if owner is not None else None) if precision == "fp8" else False
    return HstuAttentionFn.apply(q, k, v, offsets, max_len, alpha, num_targets, contextual, fp8_owner)


# --------------------------------------------------------------------------------------
# glue between the attention and the output projection
# --------------------------------------------------------------------------------------
def gate_cat_reference(u_raw, attn, weight, bias, eps: float = 1e-6):
    """``[silu(u_raw) | attn | silu(u_raw) * LayerNorm(attn)]`` with plain torch operators."""
    u = torch.nn.functional.silu(u_raw)
    n = torch.nn.functional.layer_norm(attn.float(), (attn.shape[-1],), weight.float(), bias.float(), eps).to(attn.dtype)
    return torch.cat([u, attn, u * n], dim=1)


def gate_cat_eligible(u_raw: torch.Tensor, attn: torch.Tensor) -> bool:
    D = attn.shape[-1]
    return (use_kernels(attn) and attn.dtype == torch.bfloat16 and D in (256, 512, 768) and u_raw.stride(1) == 1
            and u_raw.stride(0) % 8 == 0 and u_raw.data_ptr() % 16 == 0)


class GateCatFn(Function):
    """The concatenated input of the HSTU output projection in one pass each way (SiLU of u, layer norm
    of the attention output, their product, the concatenation, dropout of rate ``p``; backward
    recomputes all of it from ``u_raw`` and ``attn``, the dropout mask from its Philox seed).
    ``u_raw`` may be a column block of the fused uvqk projection.  The seed is drawn from torch's CPU
    generator, so ``torch.manual_seed`` fixes the masks."""

    @staticmethod
    def forward(ctx, u_raw, attn, weight, bias, eps, p=0.0):
        T, D = attn.shape
        attn = attn.contiguous()
        w, b = weight.to(torch.bfloat16).contiguous(), bias.to(torch.bfloat16).contiguous()
        cat = torch.empty((T, 3 * D), dtype=attn.dtype, device=attn.device)
        mean = torch.empty(T, dtype=torch.float32, device=attn.device)
        rstd = torch.empty(T, dtype=torch.float32, device=attn.device)
        seed = int(torch.randint(0, 2 ** 62, (1,)).item()) if p > 0 else 0
        call("b200_hstu_gate_cat_fwd", ptr(u_raw), u_raw.stride(0), ptr(attn), ptr(w), ptr(b), ptr(cat), ptr(mean), ptr(rstd),
             T, D, float(eps), float(p), seed, stream_ptr())
        ctx.save_for_backward(u_raw, attn, w, b, mean, rstd)
        ctx.refs = (weight, bias)
        ctx.drop = (float(p), seed)
        return cat

    @staticmethod
    def backward(ctx, dcat):
        from .functional import _vec_grad
        u_raw, attn, w, b, mean, rstd = ctx.saved_tensors
        T, D = attn.shape
        dcat = dcat.contiguous()
        du = torch.empty((T, D), dtype=attn.dtype, device=attn.device)
        da = torch.empty_like(attn)
        dw = torch.empty(D, dtype=torch.float32, device=attn.device)
        db = torch.empty(D, dtype=torch.float32, device=attn.device)
        scratch = torch.empty(_lib.load().b200_hstu_gate_cat_scratch_elems(T, D), dtype=torch.float32, device=attn.device)
        call("b200_hstu_gate_cat_bwd", ptr(dcat), ptr(u_raw), u_raw.stride(0), ptr(attn), ptr(w), ptr(b), ptr(mean), ptr(rstd),
             ptr(du), du.stride(0), ptr(da), ptr(dw), ptr(db), ptr(scratch), T, D, 0, ctx.drop[0], ctx.drop[1], stream_ptr())
        return du, da, _vec_grad(ctx.refs[0], dw), _vec_grad(ctx.refs[1], db), None, None


def gate_cat(u_raw, attn, weight, bias, eps: float = 1e-6, p: float = 0.0):
    if gate_cat_eligible(u_raw, attn):
        return GateCatFn.apply(u_raw, attn, weight, bias, eps, p)
    return torch.nn.functional.dropout(gate_cat_reference(u_raw, attn, weight, bias, eps), p)
