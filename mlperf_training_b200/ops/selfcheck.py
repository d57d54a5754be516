"""Start-up self-check: a handful of kernels on ramps and random operands against the eager oracle, before the clock
starts.  Every check runs the op on ``device`` tensors and on their CPU copies (the CPU branch of the same Python
function is the oracle) and compares; a failure raises - the run does not start on kernels that disagree with their
oracle (fail-closed).  On a CPU device the two sides are the same code, so the check only exercises the plumbing.

The reference does this per extension while it builds them before RUN_START: ramps, sentinel-filled outputs, a
relative-L2 guard, failure latches the feature off (generative_recommenders/ops/hip/k512_fp8_gemm.py:708-805,
generative_recommenders/ops/hip/wgrad_ck.py:439-476 ``rel_l2 <= 1e-4`` in their precision).

    python -m mlperf_training_b200.ops.selfcheck [--device cuda]
    SELF_CHECK=1 python -m mlperf_training_b200.trainer.cli ...        # the trainers call run_selfcheck() before the first step
"""
from __future__ import annotations

import argparse
import sys

import torch

from . import kernels as K
from . import mxfp8 as MX


def _rel_l2(got: torch.Tensor, want: torch.Tensor) -> float:
    g, w = got.detach().double().cpu(), want.detach().double().cpu()
    return float((g - w).norm() / w.norm().clamp(min=1e-30))


def _ramp(rows: int, cols: int, dtype, scale: float = 1.0) -> torch.Tensor:
    """Deterministic, sign-alternating ramp: every element differs, so a misplaced tile shows."""
    i = torch.arange(rows * cols, dtype=torch.float32).view(rows, cols)
    return (((i % 251) - 125.0) / 125.0 * scale * (1 - 2 * ((i // 7) % 2))).to(dtype)


def checks(dtype) -> list:
    """``[(name, fn(device) -> (got, want), tolerance)]``."""
    g = torch.Generator().manual_seed(1234)

    def gemm(dev):
        a, b = _ramp(256, 384, dtype), torch.randn(256, 384, generator=g).to(dtype) * 0.1
        return K.gemm(a.to(dev), b.to(dev)), K.gemm(a, b)

    def gemm_wgrad(dev):
        dy, x = torch.randn(256, 256, generator=g).to(dtype), _ramp(256, 384, dtype)
        return (K.gemm(dy.to(dev), x.to(dev), a_mn_major=True, b_mn_major=True, out_dtype=torch.float32),
                K.gemm(dy, x, a_mn_major=True, b_mn_major=True, out_dtype=torch.float32))

    def mx_gemm(dev):
        a, b = torch.randn(256, 512, generator=g).to(dtype), torch.randn(256, 512, generator=g).to(dtype) * 0.05
        qa, qb = MX.quantize(a.to(dev), row_tile=MX.A_TILE)[0], MX.quantize(b.to(dev), row_tile=MX.b_tile(256))[0]
        ca, cb = MX.quantize(a, row_tile=MX.A_TILE)[0], MX.quantize(b, row_tile=MX.b_tile(256))[0]
        return MX.gemm(qa, qb, out_dtype=torch.float32), MX.gemm(ca, cb, out_dtype=torch.float32)

    def rms_norm(dev):
        x, w = torch.randn(256, 512, generator=g).to(dtype), (1 + 0.1 * torch.randn(512, generator=g)).to(dtype)
        return K.norm_fwd(x.to(dev), w.to(dev), None, 1e-5, layer_norm=False)[0], K.norm_fwd(x, w, None, 1e-5, layer_norm=False)[0]

    def swiglu(dev):
        gu = torch.randn(256, 512, generator=g).to(dtype)
        return K.swiglu_fwd(gu.to(dev)), K.swiglu_fwd(gu)

    def attention(dev):
        q, k, v = (torch.randn(1, 256, h, 64, generator=g).to(dtype) for h in (4, 2, 2))
        return (K.attention_fwd(q.to(dev), k.to(dev), v.to(dev), causal=True)[0], K.attention_fwd(q, k, v, causal=True)[0])

    def cross_entropy(dev):
        logits, labels = torch.randn(256, 512, generator=g).to(dtype), torch.randint(0, 512, (256,), generator=g)
        a = K.cross_entropy_(logits.clone().to(dev), labels.to(dev), 1.0, write_grad=False)
        b = K.cross_entropy_(logits.clone(), labels, 1.0, write_grad=False)
        pick = lambda r: (r[0] if isinstance(r, (tuple, list)) else r).float().reshape(-1)
        return pick(a), pick(b)

    low = dtype == torch.bfloat16
    return [("gemm", gemm, 2e-2 if low else 1e-5), ("gemm weight-gradient form", gemm_wgrad, 2e-2 if low else 1e-5),
            ("block-scaled gemm", mx_gemm, 1e-3), ("rms norm", rms_norm, 2e-2 if low else 1e-5),
            ("swiglu", swiglu, 2e-2 if low else 1e-5), ("attention", attention, 3e-2 if low else 1e-5),
            ("cross entropy", cross_entropy, 2e-2 if low else 1e-5)]


def run_selfcheck(device="cuda", verbose: bool = False) -> dict:
    """Run every check; returns ``{name: relative L2 error}``.  Raises ``RuntimeError`` naming the checks that fail."""
    dev = torch.device(device)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    report, bad = {}, []
    for name, fn, tol in checks(dtype):
        got, want = fn(dev)
        err = _rel_l2(got, want)
        finite = bool(torch.isfinite(got.float()).all())
        report[name] = err
        if verbose:
            print(f"[selfcheck] {name}: rel_l2 {err:.3e} (limit {tol:.0e})", flush=True)
        if not finite or err > tol:
            bad.append(f"{name} (rel_l2 {err:.3e} > {tol:.0e}{'' if finite else ', non-finite output'})")
    if dev.type == "cuda":
        from . import _lib
        torch.cuda.synchronize()
        _lib.check_status("selfcheck")
    if bad:
        raise RuntimeError("kernel self-check failed: " + "; ".join(bad))
    return report


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    run_selfcheck(a.device, verbose=True)
    print("[selfcheck] ok", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
