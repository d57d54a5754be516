"""MXFP8 (e4m3 codes + one UE8M0 scale per 32 contraction elements) operands and GEMM.

``quantize`` turns a bf16 matrix into the operand copies a training step needs - the row-wise
copy (contraction along the columns) and/or the column-wise copy stored transposed (contraction
along the rows) - in one pass; ``gemm`` multiplies two such operands on the block-scaled tcgen05
tensor-core path.  On CPU tensors both run an eager emulation with identical rounding, which is the
oracle of the GPU tests.

The recipe (per-32 power-of-two scales, no amax history, no calibration, no all-reduce) is the
MX block-scaling family the reference selects for its linears
(small_llm_pretraining/primus/conf/llama3.1_8B-pretrain-fp4.yaml:108-112 ``fp4_recipe: mxfp4``;
llama2_sft/primus/src/llama2_custom.py:179-198 ``bf16_with_mxfp4_mixed``) at the MXFP8 width the
benchmark definition names.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib
from ._lib import call, ptr, stream_ptr, use_kernels

A_TILE = 128     # M tile of the GEMM: scale-atom grouping of A operands


def b_tile(n_rows: int) -> int:
    """N tile the GEMM uses for a B operand with ``n_rows`` rows (its scale-atom grouping)."""
    if _lib.LIB_PATH.exists():
        return int(_lib.load().b200_gemm_mxfp8_bn(int(n_rows)))     # the kernel's own rule
    return 208 if n_rows > 128 else 128


@dataclass
class MXOperand:
    """K-major MXFP8 operand: ``q`` ``[rows, k]`` e4m3 codes (uint8), ``sf`` scales.

    On CUDA ``sf`` is the flat atom layout for ``tile_rows``; on CPU it is a plain ``[rows, k/32]``
    uint8 matrix (biased exponents)."""
    q: torch.Tensor
    sf: torch.Tensor
    rows: int
    k: int
    tile_rows: int

    @property
    def is_cuda(self) -> bool:
        return self.q.is_cuda


def _e8m0(amax: torch.Tensor, v_max: float = 448.0) -> torch.Tensor:
    """Biased exponent of the smallest power of two s with amax / s <= v_max (448 for e4m3; 0 for amax == 0)."""
    t = (amax.float() / v_max)
    bits = t.view(torch.int32)
    e = ((bits >> 23) & 0xff) - 127
    e = e + ((bits & 0x7fffff) != 0).to(torch.int32)
    e = e.clamp(-127, 127) + 127
    return torch.where(amax > 0, e, torch.zeros_like(e)).to(torch.uint8)


def _quant_rows_cpu(x: torch.Tensor):
    """Eager row-wise MXFP8: returns (codes uint8 [R, C], sf uint8 [R, C/32])."""
    R, C = x.shape
    xb = x.float().view(R, C // 32, 32)
    sf = _e8m0(xb.abs().amax(-1))
    inv = torch.exp2(127.0 - sf.float())
    y = (xb * inv[..., None]).clamp(-448.0, 448.0)
    q = y.to(torch.float8_e4m3fn).view(torch.uint8).view(R, C)
    return q, sf


# element formats of the micro-scaled family: (mantissa bits, smallest normal exponent, largest magnitude).  Every value
# of the 4- and 6-bit formats is also an e4m3 value, so an operand rounded to one of them travels as e4m3 codes with the
# same per-32 power-of-two scales and the block-scaled GEMM multiplies it exactly: the numerics of the narrow format at
# the 8-bit operand rate.
ELEMENT_FORMATS = {"e4m3": (3, -6, 448.0), "e3m2": (2, -2, 28.0), "e2m3": (3, 0, 7.5), "e2m1": (1, 0, 6.0)}


def round_to_format(y: torch.Tensor, fmt: str, stochastic: bool = False) -> torch.Tensor:
    """``y`` (fp32) rounded to the nearest value of ``fmt`` (ties to even; saturating), or rounded stochastically:
    up with the probability of the distance to the lower neighbour, so that the expectation is ``y``."""
    m_bits, e_min, v_max = ELEMENT_FORMATS[fmt]
    a = y.abs().clamp(max=v_max)
    _, ex = torch.frexp(a)                                   # a = m * 2^ex with m in [0.5, 1)
    quantum = torch.exp2((ex - 1).clamp(min=e_min).float() - m_bits)
    t = a / quantum
    r = torch.floor(t + torch.rand_like(t)) if stochastic else torch.round(t)
    return torch.copysign((r * quantum).clamp(max=v_max), y)


def quantize_rows_narrow(x: torch.Tensor, fmt: str, tile_rows: int, stochastic: bool = False) -> MXOperand:
    """Row-wise micro-scaled operand of ``x [R, C]`` with elements rounded to ``fmt`` (one power-of-two scale per 32
    contraction elements, chosen so that the block's largest magnitude fits the format), stored as e4m3 codes.  Runs as
    tensor operations on either device; on CUDA the scales go into the atom layout the GEMM reads."""
    R, C = x.shape
    if C % 32:
        raise ValueError(f"quantize_rows_narrow: {C} columns are not a multiple of 32")
    v_max = ELEMENT_FORMATS[fmt][2]
    xb = x.float().view(R, C // 32, 32)
    sf = _e8m0(xb.abs().amax(-1), v_max)
    y = round_to_format(xb * torch.exp2(127.0 - sf.float())[..., None], fmt, stochastic)
    q = y.to(torch.float8_e4m3fn).view(torch.uint8).view(R, C)
    if x.is_cuda:
        buf = torch.zeros(sf_bytes(R, C, tile_rows), dtype=torch.uint8, device=x.device)
        buf[sf_index(R, C, tile_rows, x.device)] = sf
        sf = buf
    return MXOperand(q, sf, R, C, tile_rows)


def sf_index(rows: int, k: int, tile_rows: int, device) -> torch.Tensor:
    """Flat byte offsets, shape ``[rows, k/32]``, of every scale in the atom layout."""
    r = torch.arange(rows, device=device, dtype=torch.int64)[:, None]
    kc = torch.arange(k // 32, device=device, dtype=torch.int64)[None, :]
    atoms = (tile_rows + 127) // 128
    tile = r // tile_rows
    rr = r - tile * tile_rows
    atom, ra = rr // 128, rr % 128
    return ((tile * ((k + 127) // 128) + kc // 4) * atoms + atom) * 512 + (ra % 32) * 16 + (ra // 32) * 4 + (kc % 4)


def sf_bytes(rows: int, k: int, tile_rows: int) -> int:
    tiles = (rows + tile_rows - 1) // tile_rows
    return tiles * ((k + 127) // 128) * ((tile_rows + 127) // 128) * 512


def sf_plain(op: MXOperand) -> torch.Tensor:
    """Scales of ``op`` as a plain ``[rows, k/32]`` uint8 matrix (un-swizzles the CUDA layout)."""
    if not op.is_cuda:
        return op.sf
    return op.sf[sf_index(op.rows, op.k, op.tile_rows, op.sf.device)]


def dequantize(op: MXOperand) -> torch.Tensor:
    """fp32 ``[rows, k]`` value of an operand."""
    q = op.q.view(torch.float8_e4m3fn).float().view(op.rows, op.k // 32, 32)
    s = torch.exp2(sf_plain(op).float() - 127.0)
    return (q * s[..., None]).view(op.rows, op.k)


def quantize(x: torch.Tensor, *, row_tile: int | None = None, col_tile: int | None = None, fmt: str = "e4m3",
             col_fmt: str | None = None, stochastic: bool = False):
    """bf16 ``x`` ``[R, C]`` -> ``(row_op, col_op)``.  ``fmt`` / ``col_fmt`` (default: ``fmt``): element format of the
    row-wise / column-wise copy; anything but round-to-nearest e4m3 goes through ``quantize_rows_narrow``.

    ``row_op`` (when ``row_tile`` is given) has rows = R, contraction = C; ``col_op`` (when
    ``col_tile`` is given) is the transposed copy with rows = C, contraction = R.  The tile
    arguments say how the consuming GEMM tiles the operand's rows: ``A_TILE`` for an A operand,
    ``b_tile(rows)`` for a B operand.  R must be a multiple of 128 and C of 32."""
    R, C = x.shape
    if R % 128 or C % 32:
        raise ValueError(f"mxfp8.quantize: shape {R}x{C}: rows must be a multiple of 128, columns of 32")
    col_fmt = col_fmt or fmt
    if stochastic or fmt != "e4m3" or col_fmt != "e4m3":
        row_op = quantize_rows_narrow(x, fmt, row_tile, stochastic) if row_tile is not None else None
        col_op = quantize_rows_narrow(x.t().contiguous(), col_fmt, col_tile, stochastic) if col_tile is not None else None
        return row_op, col_op
    if not use_kernels(x):
        row_op = col_op = None
        if row_tile is not None:
            q, sf = _quant_rows_cpu(x)
            row_op = MXOperand(q, sf, R, C, row_tile)
        if col_tile is not None:
            q, sf = _quant_rows_cpu(x.t().contiguous())
            col_op = MXOperand(q, sf, C, R, col_tile)
        return row_op, col_op
    if x.dtype != torch.bfloat16:
        raise TypeError("mxfp8.quantize: bf16 input required")
    if x.stride(1) != 1 or (x.stride(0) * 2) % 16 or x.data_ptr() % 16:
        x = x.contiguous()
    q_row, sf_row, q_col, sf_col = _alloc_ops(R, C, row_tile, col_tile, x.device)
    call("b200_quant_mxfp8", ptr(x), x.stride(0), R, C, ptr(q_row), ptr(sf_row), row_tile or 0, ptr(q_col),
         ptr(sf_col), col_tile or 0, stream_ptr())
    row_op = MXOperand(q_row, sf_row, R, C, row_tile) if row_tile is not None else None
    col_op = MXOperand(q_col, sf_col, C, R, col_tile) if col_tile is not None else None
    return row_op, col_op


def _sf_buffer(rows: int, k: int, tile: int, dev) -> torch.Tensor:
    """Scale buffer of an operand; zero-filled when the quantiser leaves padding rows of an atom unwritten."""
    n = sf_bytes(rows, k, tile)
    if tile % 128 or rows % 128:
        return torch.zeros(n, dtype=torch.uint8, device=dev)
    return torch.empty(n, dtype=torch.uint8, device=dev)


def _alloc_ops(R: int, C: int, row_tile, col_tile, dev):
    q_row = sf_row = q_col = sf_col = None
    if row_tile is not None:
        q_row = torch.empty((R, C), dtype=torch.uint8, device=dev)
        sf_row = _sf_buffer(R, C, row_tile, dev)
    if col_tile is not None:
        q_col = torch.empty((C, R), dtype=torch.uint8, device=dev)
        sf_col = _sf_buffer(C, R, col_tile, dev)
    return q_row, sf_row, q_col, sf_col


def quantize_swiglu(gu: torch.Tensor, *, row_tile: int | None = None, col_tile: int | None = None):
    """Quantised ``a = silu(gate) * up`` of ``gu [R, 2F]`` (gate columns first) without materialising
    ``a``: same return value as ``quantize(swiglu(gu), ...)``."""
    R, F2 = gu.shape
    F = F2 // 2
    if not use_kernels(gu):
        from . import kernels as K
        return quantize(K.swiglu_fwd(gu), row_tile=row_tile, col_tile=col_tile)
    if gu.stride(1) != 1 or (gu.stride(0) * 2) % 16 or gu.data_ptr() % 16:
        gu = gu.contiguous()
    q_row, sf_row, q_col, sf_col = _alloc_ops(R, F, row_tile, col_tile, gu.device)
    call("b200_quant_swiglu_mxfp8", ptr(gu), gu.stride(0), R, F, ptr(q_row), ptr(sf_row), row_tile or 0, ptr(q_col),
         ptr(sf_col), col_tile or 0, stream_ptr())
    return (MXOperand(q_row, sf_row, R, F, row_tile) if row_tile is not None else None,
            MXOperand(q_col, sf_col, F, R, col_tile) if col_tile is not None else None)


def quantize_swiglu_bwd(da: torch.Tensor, gu: torch.Tensor, *, row_tile: int | None = None, col_tile: int | None = None):
    """Quantised ``dgu [R, 2F]`` (d gate | d up) from ``da [R, F]`` and ``gu [R, 2F]`` without
    materialising it: same return value as ``quantize(swiglu_bwd(da, gu), ...)``."""
    R, F2 = gu.shape
    F = F2 // 2
    if not use_kernels(gu) or F % 128:      # the fused kernel's tiles must not straddle the gate | up boundary
        from . import kernels as K
        return quantize(K.swiglu_bwd(da, gu), row_tile=row_tile, col_tile=col_tile)
    da = da if (da.stride(1) == 1 and (da.stride(0) * 2) % 16 == 0 and da.data_ptr() % 16 == 0) else da.contiguous()
    if gu.stride(1) != 1 or (gu.stride(0) * 2) % 16 or gu.data_ptr() % 16:
        gu = gu.contiguous()
    q_row, sf_row, q_col, sf_col = _alloc_ops(R, F2, row_tile, col_tile, gu.device)
    call("b200_quant_swiglu_bwd_mxfp8", ptr(da), da.stride(0), ptr(gu), gu.stride(0), R, F, ptr(q_row), ptr(sf_row),
         row_tile or 0, ptr(q_col), ptr(sf_col), col_tile or 0, stream_ptr())
    return (MXOperand(q_row, sf_row, R, F2, row_tile) if row_tile is not None else None,
            MXOperand(q_col, sf_col, F2, R, col_tile) if col_tile is not None else None)


def gemm(a: MXOperand, b: MXOperand, *, out: torch.Tensor | None = None, out_dtype=torch.bfloat16,
         accumulate: bool = False, bias: torch.Tensor | None = None, residual: torch.Tensor | None = None,
         alpha: float = 1.0) -> torch.Tensor:
    """``D[M,N] (+)= alpha * deq(a) @ deq(b)^T (+ bias) (+ residual)``."""
    if a.k != b.k:
        raise ValueError(f"mxfp8.gemm: contraction mismatch {a.k} vs {b.k}")
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
    if a.tile_rows != A_TILE or b.tile_rows != b_tile(N):
        raise ValueError(f"mxfp8.gemm: operand scale tiling ({a.tile_rows}, {b.tile_rows}) does not match the "
                         f"kernel tiles ({A_TILE}, {b_tile(N)})")
    if out is None:
        if accumulate:
            raise ValueError("mxfp8.gemm: accumulate needs an output tensor")
        out = torch.empty((M, N), dtype=out_dtype, device=a.q.device)
    if out.dtype not in (torch.bfloat16, torch.float32) or out.stride(1) != 1:
        raise TypeError("mxfp8.gemm: output must be row-major bf16 or fp32")
    if (out.stride(0) * out.element_size()) % 16 or out.data_ptr() % 16:
        raise ValueError("mxfp8.gemm: output pitch/base must be 16-byte aligned")
    if bias is not None:
        bias = bias.to(torch.bfloat16).contiguous()
    ldr = 0
    if residual is not None:
        if residual.dtype != torch.bfloat16 or residual.stride(1) != 1:
            residual = residual.to(torch.bfloat16).contiguous()
        ldr = residual.stride(0)
    call("b200_gemm_mxfp8", ptr(a.q), ptr(a.sf), ptr(b.q), ptr(b.sf), ptr(out), M, N, Kd, a.q.stride(0),
         b.q.stride(0), out.stride(0), int(out.dtype == torch.float32), int(accumulate), ptr(bias), ptr(residual),
         ldr, float(alpha), stream_ptr())
    return out
