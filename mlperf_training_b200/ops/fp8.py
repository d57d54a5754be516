"""Per-tensor FP8 operands (e4m3 / e5m2 codes with ONE scale factor per tensor), delayed scaling, GEMM.

The second low-precision recipe of the package, next to MXFP8 (``ops.mxfp8``): forward operands
(activations, weights) are e4m3, gradients e5m2 ("hybrid"), each tensor scaled by
``fmax / amax`` where ``amax`` comes from a short history of earlier steps (delayed scaling), so no
reduction has to finish before the cast.  The quantiser writes the absolute maximum it saw into a
device word; ``DelayedScale.roll`` turns the history into the next factor on the device - the host
never reads an amax.  This is the recipe of the reference's recommender FP8 path
(generative_recommenders/ops/triton/triton_fp8.py: per-tensor e4m3 with calibrate-then-freeze factors;
generative_recommenders/ops/triton/bwd_fp8.py: e5m2 gradients, delayed factor refreshed on a cadence)
and of the FP8 phase the FLUX forward switches to (flux1/primus/patches/flux_fprop_switch.py:36-279).

On CPU tensors the same functions run an eager emulation with ``torch.float8_*`` casts (the oracle of
the GPU tests).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib
from ._lib import call, ptr, stream_ptr, use_kernels

FMAX = {"e4m3": 448.0, "e5m2": 57344.0}
_TORCH = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}


# How a site's scale follows the tensor, per element format (``set_policy`` changes it for sites created afterwards):
#   mode "rolling": the factor follows the maximum of the last ``history`` epochs (delayed scaling);
#   mode "frozen":  ``history`` calibration epochs, then the factor never moves again (the recommender's forward sites:
#                   4 steps, margin 1.5, generative_recommenders/ops/triton/triton_fp8.py:94-102,694-749);
#   ``refresh``:    a rolling factor is republished only every ``refresh`` epochs from the maximum collected since
#                   (the recommender's gradient sites: every 200 calls, margin 8, .../bwd_fp8.py:157-169,1073-1154);
#   ``margin``:     headroom multiplier on the collected maximum.
SCALE_POLICY = {"e4m3": dict(mode="rolling", history=4, margin=1.0, refresh=1),
                "e5m2": dict(mode="rolling", history=4, margin=1.0, refresh=1)}


def set_policy(fmt: str, **kw) -> dict:
    """Change the scale policy of ``fmt`` sites created from now on; returns the previous policy."""
    old = dict(SCALE_POLICY[fmt])
    bad = set(kw) - set(old)
    if bad or kw.get("mode", old["mode"]) not in ("rolling", "frozen"):
        raise ValueError(f"fp8 scale policy: unknown setting {sorted(bad) or kw.get('mode')}")
    SCALE_POLICY[fmt].update(kw)
    return old


@dataclass
class FP8Operand:
    """K-major operand: ``q [rows, k]`` codes (uint8) and ``inv_scale`` (one fp32, on the device):
    value = code * inv_scale."""
    q: torch.Tensor
    inv_scale: torch.Tensor
    rows: int
    k: int
    fmt: str

    @property
    def is_cuda(self) -> bool:
        return self.q.is_cuda


class DelayedScale:
    """Scale state of one tensor site (an activation, a weight, a gradient of one linear).

    ``scale`` multiplies the tensor before the cast; ``amax`` collects max(|x|) of the current epoch
    (bit pattern of a non-negative float, so an integer atomic max orders it).  ``roll`` - called when
    the optimizer has stepped - pushes the collected amax into the history and recomputes ``scale`` =
    ``fmax / (max(history) * 2^margin)``, all on the device."""

    def __init__(self, fmt: str, device, history: int | None = None, margin: int = 0):
        pol = SCALE_POLICY[fmt]
        self.fmt, self.margin = fmt, margin
        self.mode, self.margin_mult, self.refresh = pol["mode"], float(pol["margin"]), max(int(pol["refresh"]), 1)
        self.hist = torch.zeros(history if history is not None else int(pol["history"]), dtype=torch.float32, device=device)
        self.amax = torch.zeros(1, dtype=torch.int32, device=device)
        self.scale = torch.ones(1, dtype=torch.float32, device=device)
        self.inv_scale = torch.ones(1, dtype=torch.float32, device=device)
        self.epoch = None
        self.pos = 0
        self.primed = False
        self.frozen = False

    def _set_from(self, amax: torch.Tensor) -> None:
        a = amax.float().clamp_min(1e-30) * (2.0 ** self.margin) * self.margin_mult
        self.scale.copy_((FMAX[self.fmt] / a).reshape(1))
        self.inv_scale.copy_((a / FMAX[self.fmt]).reshape(1))

    def prepare(self, x: torch.Tensor, epoch: int) -> None:
        """Make ``scale`` valid for quantising ``x`` in ``epoch``."""
        if self.frozen:
            return
        if not self.primed:
            # no history yet: this tensor's own maximum (one extra pass, first use only)
            self._set_from(x.detach().abs().amax())
            self.primed, self.epoch = True, epoch
            return
        if epoch != self.epoch:
            self.epoch = epoch
            if self.refresh > 1:
                # the collected maximum keeps growing over the window; it is published at the window's end
                self.pos += 1
                if self.pos % self.refresh:
                    return
                self.hist[(self.pos // self.refresh) % self.hist.numel()] = self.amax.view(torch.float32)[0]
            else:
                self.hist[self.pos % self.hist.numel()] = self.amax.view(torch.float32)[0]
                self.pos += 1
            self.amax.zero_()
            self._set_from(self.hist.max())
            if self.mode == "frozen" and self.pos >= self.hist.numel():
                self.frozen = True                       # calibration complete: the factor stays

    def state_dict(self) -> dict:
        return {"fmt": self.fmt, "hist": self.hist.detach().cpu(), "amax": self.amax.detach().cpu(), "scale": self.scale.detach().cpu(),
                "inv_scale": self.inv_scale.detach().cpu(), "epoch": self.epoch, "pos": self.pos, "primed": self.primed,
                "frozen": self.frozen}

    def load_state_dict(self, sd: dict) -> None:
        for k in ("hist", "amax", "scale", "inv_scale"):
            getattr(self, k).copy_(sd[k])
        self.epoch, self.pos, self.primed, self.frozen = sd["epoch"], int(sd["pos"]), bool(sd["primed"]), bool(sd["frozen"])


def quantize(x: torch.Tensor, state: DelayedScale, *, want_row: bool = True, want_col: bool = False):
    """bf16 ``x [R, C]`` -> ``(row_op, col_op)``: ``row_op`` has rows R and contraction C, ``col_op`` is
    the transposed copy (rows C, contraction R).  ``state.scale`` is applied; the tensor's amax is
    accumulated into ``state.amax``.  R and C must be multiples of 128 on CUDA."""
    R, C = x.shape
    fmt = state.fmt
    if not use_kernels(x):
        y = (x.float() * state.scale.to(x.device)).clamp(-FMAX[fmt], FMAX[fmt]).to(_TORCH[fmt])
        cur = x.detach().abs().amax().float().reshape(1)
        state.amax.copy_(torch.maximum(state.amax.view(torch.float32), cur).view(torch.int32))
        q = y.view(torch.uint8)
        row = FP8Operand(q, state.inv_scale, R, C, fmt) if want_row else None
        col = FP8Operand(q.t().contiguous(), state.inv_scale, C, R, fmt) if want_col else None
        return row, col
    if R % 128 or C % 128:
        raise ValueError(f"fp8.quantize: shape {R}x{C} must be a multiple of 128 in both dims")
    if x.dtype != torch.bfloat16:
        raise TypeError("fp8.quantize: bf16 input required")
    if x.stride(1) != 1 or (x.stride(0) * 2) % 16 or x.data_ptr() % 16:
        x = x.contiguous()
    q_row = torch.empty((R, C), dtype=torch.uint8, device=x.device) if want_row else None
    q_col = torch.empty((C, R), dtype=torch.uint8, device=x.device) if want_col else None
    call("b200_quant_fp8", ptr(x), x.stride(0), R, C, ptr(state.scale), int(fmt == "e5m2"), ptr(q_row), ptr(q_col),
         ptr(state.amax), stream_ptr())
    return (FP8Operand(q_row, state.inv_scale, R, C, fmt) if want_row else None,
            FP8Operand(q_col, state.inv_scale, C, R, fmt) if want_col else None)


def quantize_rows(x: torch.Tensor, state: DelayedScale) -> FP8Operand:
    """Row-wise copy of a 2-D bf16 ``x [R, C]`` with any number of rows (jagged token buffers; ``x`` may be a
    column block of a wider matrix): codes ``[R, C]``, ``state.scale`` applied, amax accumulated."""
    R, C = x.shape
    fmt = state.fmt
    if not use_kernels(x):
        return quantize(x, state)[0]
    if x.dtype != torch.bfloat16:
        raise TypeError("fp8.quantize_rows: bf16 input required")
    if x.stride(1) != 1 or x.stride(0) % 8 or x.data_ptr() % 16:
        x = x.contiguous()
    q = torch.empty((R, C), dtype=torch.uint8, device=x.device)
    call("b200_quant_fp8_rows", ptr(x), x.stride(0), R, C, ptr(state.scale), int(fmt == "e5m2"), ptr(q), q.stride(0),
         ptr(state.amax), stream_ptr())
    return FP8Operand(q, state.inv_scale, R, C, fmt)


def dequantize(op: FP8Operand) -> torch.Tensor:
    return op.q.view(_TORCH[op.fmt]).float() * op.inv_scale.to(op.q.device)


def gemm(a: FP8Operand, b: FP8Operand, *, out: torch.Tensor | None = None, out_dtype=torch.bfloat16,
         accumulate: bool = False, bias: torch.Tensor | None = None, residual: torch.Tensor | None = None,
         alpha: float = 1.0) -> torch.Tensor:
    """``D[M,N] (+)= alpha * deq(a) @ deq(b)^T (+ bias) (+ residual)``."""
    if a.k != b.k:
        raise ValueError(f"fp8.gemm: contraction mismatch {a.k} vs {b.k}")
    M, N, Kd = a.rows, b.rows, a.k
    if out is not None:
        out_dtype = out.dtype
    if not a.is_cuda:
        d = alpha * (dequantize(a) @ dequantize(b).t())
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
    _lib.require()
    if out is None:
        if accumulate:
            raise ValueError("fp8.gemm: accumulate needs an output tensor")
        out = torch.empty((M, N), dtype=out_dtype, device=a.q.device)
    if out.dtype not in (torch.bfloat16, torch.float32) or out.stride(1) != 1:
        raise TypeError("fp8.gemm: output must be row-major bf16 or fp32")
    if bias is not None:
        bias = bias.to(torch.bfloat16).contiguous()
    ldr = 0
    if residual is not None:
        if residual.dtype != torch.bfloat16 or residual.stride(1) != 1:
            residual = residual.to(torch.bfloat16).contiguous()
        ldr = residual.stride(0)
    call("b200_gemm_fp8", ptr(a.q), ptr(b.q), ptr(out), M, N, Kd, a.q.stride(0), b.q.stride(0), out.stride(0),
         int(a.fmt == "e5m2"), int(b.fmt == "e5m2"), ptr(a.inv_scale), ptr(b.inv_scale), int(out.dtype == torch.float32),
         int(accumulate), ptr(bias), ptr(residual), ldr, float(alpha), stream_ptr())
    return out
