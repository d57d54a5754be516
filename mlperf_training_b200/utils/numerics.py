"""Numerics probes for the block-scaled FP8 linears: signal-to-noise ratio and cosine of each GEMM of
a linear layer (forward, data gradient, weight gradient) computed from MXFP8-quantised operands,
against the same products in fp64.

    python -m mlperf_training_b200.utils.numerics [--tokens 512 --in 1024 --out 1024 --outliers 0.001]
    python -m mlperf_training_b200.utils.numerics --precision mxfp4 a6w4 fp8      # through the training path itself

``linear_site_report(x, w, dy)`` quantises exactly as the training path does (e4m3 values with one
power-of-two scale per 32 elements along the contraction dimension of each GEMM: rows of x and w
for the forward product, columns for the two gradient products), dequantises, multiplies in fp64
and compares.  ``recipe_report(x, w, dy, precision)`` runs the linear triple of the training path itself (forward,
data gradient, weight gradient under ``precision``: any micro-scaled recipe or per-tensor fp8, with its stochastic
rounding and Hadamard operands) and compares each result with fp64.  Both run on CPU or GPU tensors.  The reference carries the same kind of probe for its FP8
paths (generative_recommenders/ops/triton/fp8_wgrad_snr.py, preproc_fp8_snr.py: fp64 reference GEMMs,
SNR and cosine per site).
"""
from __future__ import annotations

import argparse
import json
import math
import sys

import torch

from ..ops import mxfp8 as MX


def snr_db(ref: torch.Tensor, got: torch.Tensor) -> float:
    """10 log10(|ref|^2 / |ref - got|^2) in fp64; inf when identical."""
    r, g = ref.double(), got.double()
    noise = float(((r - g) ** 2).sum())
    sig = float((r ** 2).sum())
    if noise == 0.0:
        return math.inf
    return 10.0 * math.log10(max(sig, 1e-300) / noise)


def cosine(ref: torch.Tensor, got: torch.Tensor) -> float:
    r, g = ref.double().flatten(), got.double().flatten()
    return float((r @ g) / (r.norm() * g.norm()).clamp(min=1e-300))


def _mx(x: torch.Tensor, along_rows: bool) -> torch.Tensor:
    """``x`` after a round trip through MXFP8 with the 32-element blocks along its rows (contraction =
    last dim) or along its columns (contraction = first dim), as fp64."""
    x = x.to(torch.bfloat16).contiguous()
    row_op, col_op = MX.quantize(x, row_tile=128 if along_rows else None, col_tile=None if along_rows else 128)
    if along_rows:
        return MX.dequantize(row_op).double()
    return MX.dequantize(col_op).double().t()


def linear_site_report(x: torch.Tensor, w: torch.Tensor, dy: torch.Tensor) -> dict:
    """``x [T, K]``, ``w [N, K]``, ``dy [T, N]`` (all dims multiples of 128).  Returns SNR (dB) and cosine
    of ``y = x w^T`` (blocks along K), ``dx = dy w`` (blocks along N) and ``dw = dy^T x`` (blocks along T)."""
    xb, wb, db = (t.to(torch.bfloat16).double() for t in (x, w, dy))
    sites = {
        "fwd": (xb @ wb.t(), _mx(x, True) @ _mx(w, True).t()),
        "dgrad": (db @ wb, _mx(dy, True) @ _mx(w, False)),
        "wgrad": (db.t() @ xb, _mx(dy, False).t() @ _mx(x, False)),
    }
    return {k: {"snr_db": round(snr_db(r, g), 2), "cosine": round(cosine(r, g), 6)} for k, (r, g) in sites.items()}


def recipe_report(x: torch.Tensor, w: torch.Tensor, dy: torch.Tensor, precision: str) -> dict:
    """SNR (dB) and cosine of ``y``, ``dx`` and ``dw`` as the training path computes them under ``precision``."""
    from ..ops import functional as F
    dt = torch.bfloat16 if x.is_cuda else torch.float32
    xq = x.to(dt).detach().clone().requires_grad_(True)
    wq = w.to(dt).detach().clone().requires_grad_(True)
    y = F.linear(xq, wq, None, None, precision)
    y.backward(dy.to(dt))
    xb, wb, db = (t.to(dt).double() for t in (x, w, dy))
    sites = {"fwd": (xb @ wb.t(), y.detach()), "dgrad": (db @ wb, xq.grad), "wgrad": (db.t() @ xb, wq.grad)}
    return {k: {"snr_db": round(snr_db(r, g), 2), "cosine": round(cosine(r, g), 6)} for k, (r, g) in sites.items()}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--in", dest="k", type=int, default=1024)
    ap.add_argument("--out", dest="n", type=int, default=1024)
    ap.add_argument("--outliers", type=float, default=0.0, help="fraction of activation entries multiplied by 50")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--precision", nargs="*", default=[], help="recipes to run through the training path (mxfp8 mxfp6 mxfp4 a6w4 fp8 ...)")
    a = ap.parse_args(argv)
    g = torch.Generator().manual_seed(a.seed)
    x = torch.randn(a.tokens, a.k, generator=g)
    if a.outliers > 0:
        x = torch.where(torch.rand(x.shape, generator=g) < a.outliers, x * 50, x)
    w = torch.randn(a.n, a.k, generator=g) * 0.02
    dy = torch.randn(a.tokens, a.n, generator=g) * 1e-3
    print(json.dumps({"shape": [a.tokens, a.k, a.n], "outliers": a.outliers, **linear_site_report(x, w, dy)}))
    for prec in a.precision:
        print(json.dumps({"precision": prec, **recipe_report(x, w, dy, prec)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
