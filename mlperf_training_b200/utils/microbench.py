"""Kernel micro-benchmarks: device-timed (CUDA events) throughput of the library's hot kernels,
each next to the stock library call for the same problem (cuBLAS through ``torch.matmul``,
``scaled_dot_product_attention``), with an L2 flush between timed launches.

    python -m mlperf_training_b200.utils.microbench gemm mxfp8 fp8 attention elementwise grouped hstu glue sparse comm [--quick]

Prints one JSON object per measurement.
"""
from __future__ import annotations

import argparse
import json
import math
import sys

import torch

from ..ops import _lib, kernels

_FLUSH = None


def flush_l2() -> None:
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _FLUSH.zero_()


ITERS = 10
WARMUP = 3


def time_ms(fn, iters: int | None = None, warmup: int | None = None) -> float:
    """Median device time of ``fn`` in milliseconds, L2 flushed before every timed launch."""
    iters = ITERS if iters is None else min(iters, ITERS)
    warmup = WARMUP if warmup is None else min(warmup, WARMUP)
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def emit(**kw) -> None:
    print(json.dumps(kw), flush=True)


GEMM_SHAPES = [
    # (M, N, K, a_mn, b_mn, tag)
    (8192, 6144, 4096, False, False, "llama8b qkv fwd"),
    (8192, 4096, 4096, False, False, "llama8b proj fwd"),
    (8192, 28672, 4096, False, False, "llama8b gate_up fwd"),
    (8192, 4096, 14336, False, False, "llama8b down fwd"),
    (8192, 4096, 28672, False, True, "llama8b gate_up dgrad"),
    (28672, 4096, 8192, True, True, "llama8b gate_up wgrad"),
    (8192, 14336, 4096, False, True, "llama8b down dgrad"),
    (4096, 14336, 8192, True, True, "llama8b down wgrad"),
    (8192, 128256, 4096, False, False, "llama8b lm_head fwd"),
    (8192, 8192, 8192, False, False, "square 8192"),
]


def bench_gemm(quick: bool) -> None:
    shapes = GEMM_SHAPES[:3] + GEMM_SHAPES[-1:] if quick else GEMM_SHAPES
    for M, N, K, a_mn, b_mn, tag in shapes:
        a = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
        b = torch.randn((K, N) if b_mn else (N, K), device="cuda").bfloat16()
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms = time_ms(lambda: kernels.gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn, out=out))
        am = a.t() if a_mn else a
        bm = b if b_mn else b.t()
        ms_ref = time_ms(lambda: torch.matmul(am, bm, out=out))
        fl = 2.0 * M * N * K
        emit(kernel="gemm_bf16", tag=tag, M=M, N=N, K=K, a_mn=a_mn, b_mn=b_mn, ms=round(ms, 4),
             tflops=round(fl / ms / 1e9, 1), cublas_ms=round(ms_ref, 4), cublas_tflops=round(fl / ms_ref / 1e9, 1))
        _lib.check_status(tag)
        del a, b, out


def bench_mxfp8(quick: bool) -> None:
    from ..ops import mxfp8
    shapes = [(M, N, K, tag) for (M, N, K, a_mn, b_mn, tag) in GEMM_SHAPES if not a_mn and not b_mn]
    for M, N, K, tag in (shapes[:3] if quick else shapes):
        a = torch.randn(M, K, device="cuda").bfloat16()
        b = torch.randn(N, K, device="cuda").bfloat16()
        ms_q = time_ms(lambda: mxfp8.quantize(a, row_tile=mxfp8.A_TILE, col_tile=mxfp8.b_tile(K)))
        a_op, _ = mxfp8.quantize(a, row_tile=mxfp8.A_TILE)
        b_op, _ = mxfp8.quantize(b, row_tile=mxfp8.b_tile(N))
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms = time_ms(lambda: mxfp8.gemm(a_op, b_op, out=out))
        fl = 2.0 * M * N * K
        lib = {}
        try:
            # the library's block-scaled GEMM on the same codes (cuBLASLt through torch._scaled_mm, unit scales:
            # a timing reference only)
            e8 = torch.float8_e8m0fnu
            sa = torch.full((M * (K // 32),), 127, dtype=torch.uint8, device="cuda").view(e8)
            sb = torch.full((N * (K // 32),), 127, dtype=torch.uint8, device="cuda").view(e8)
            qa, qb = a_op.q.view(torch.float8_e4m3fn), b_op.q.view(torch.float8_e4m3fn)
            f = lambda: torch._scaled_mm(qa, qb.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)
            ms_l = time_ms(f)
            lib = {"cublaslt_mx_ms": round(ms_l, 4), "cublaslt_mx_tflops": round(fl / ms_l / 1e9, 1)}
        except Exception as e:  # this torch build has no MX scaled_mm for the shape
            lib = {"cublaslt_mx_error": str(e)[:100]}
        emit(kernel="gemm_mxfp8", tag=tag, M=M, N=N, K=K, ms=round(ms, 4), tflops=round(fl / ms / 1e9, 1),
             quant_dual_ms=round(ms_q, 4), quant_gbs=round(M * K * 4.06 / ms_q / 1e6, 1), **lib)
        _lib.check_status(tag)
        del a, b, out, a_op, b_op
    # the quantisers that carry SwiGLU and its backward (Llama-3.1-8B MLP width)
    R, F = 8192, (4096 if quick else 14336)
    gu = torch.randn(R, 2 * F, device="cuda").bfloat16()
    da = torch.randn(R, F, device="cuda").bfloat16()
    ms1 = time_ms(lambda: mxfp8.quantize_swiglu(gu, row_tile=mxfp8.A_TILE, col_tile=mxfp8.b_tile(F)))
    emit(kernel="quant_swiglu_mxfp8", R=R, F=F, ms=round(ms1, 4), gbs=round(R * F * (4 + 2.06) / ms1 / 1e6, 1))
    ms2 = time_ms(lambda: mxfp8.quantize_swiglu_bwd(da, gu, row_tile=mxfp8.A_TILE, col_tile=mxfp8.A_TILE))
    emit(kernel="quant_swiglu_bwd_mxfp8", R=R, F=F, ms=round(ms2, 4), gbs=round(R * F * (6 + 4.12) / ms2 / 1e6, 1))
    _lib.check_status("quant swiglu")
    del gu, da


ATTN_SHAPES = [
    # B, S, Hq, Hkv, D, causal, window, tag
    (1, 8192, 32, 8, 128, True, 0, "llama8b"),
    (1, 8192, 64, 8, 64, True, 0, "gpt-oss full"),
    (1, 8192, 64, 8, 64, True, 128, "gpt-oss window"),
    (32, 512, 24, 24, 128, False, 0, "flux joint"),
]


def bench_attention(quick: bool) -> None:
    for B, S, Hq, Hkv, D, causal, window, tag in (ATTN_SHAPES[:1] if quick else ATTN_SHAPES):
        q = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
        k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
        v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
        do = torch.randn_like(q)
        pairs = S * S / 2 if causal else S * S
        if window:
            pairs = S * window
        fl_fwd = 4.0 * B * Hq * pairs * D
        o, lse = kernels.attention_fwd(q, k, v, causal=causal, window=window)
        ms_f = time_ms(lambda: kernels.attention_fwd(q, k, v, causal=causal, window=window))
        ms_b = time_ms(lambda: kernels.attention_bwd(do, q, k, v, o, lse, causal=causal, window=window))
        ref = {}
        if not window:
            qt, kt, vt = (t.transpose(1, 2) for t in (q, k, v))
            f = lambda: torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, is_causal=causal,
                                                                         enable_gqa=True)
            try:
                ref["sdpa_fwd_ms"] = round(time_ms(f), 4)
                ref["sdpa_fwd_tflops"] = round(fl_fwd / ref["sdpa_fwd_ms"] / 1e9, 1)
            except Exception as e:  # library path unavailable for this shape
                ref["sdpa_error"] = str(e)[:80]
        emit(kernel="attention", tag=tag, B=B, S=S, Hq=Hq, Hkv=Hkv, D=D, causal=causal, window=window,
             fwd_ms=round(ms_f, 4), fwd_tflops=round(fl_fwd / ms_f / 1e9, 1), bwd_ms=round(ms_b, 4),
             bwd_tflops=round(2.5 * fl_fwd / ms_b / 1e9, 1), **ref)
        _lib.check_status(tag)


def bench_elementwise(quick: bool) -> None:
    T, D, Fh, V = 8192, 4096, 14336, 128256
    x = torch.randn(T, D, device="cuda").bfloat16()
    w = torch.ones(D, device="cuda").bfloat16()
    ms = time_ms(lambda: kernels.norm_fwd(x, w, None, 1e-5))
    emit(kernel="rmsnorm_fwd", T=T, D=D, ms=round(ms, 4), gbs=round(2 * x.numel() * 2 / ms / 1e6, 1))
    y, h, mean, rstd = kernels.norm_fwd(x, w, None, 1e-5)
    ms = time_ms(lambda: kernels.norm_bwd(x, h, w, None, mean, rstd))
    emit(kernel="rmsnorm_bwd", T=T, D=D, ms=round(ms, 4), gbs=round(3 * x.numel() * 2 / ms / 1e6, 1))
    gu = torch.randn(T, 2 * Fh, device="cuda").bfloat16()
    ms = time_ms(lambda: kernels.swiglu_fwd(gu))
    emit(kernel="swiglu_fwd", T=T, F=Fh, ms=round(ms, 4), gbs=round(3 * T * Fh * 2 / ms / 1e6, 1))
    da = torch.randn(T, Fh, device="cuda").bfloat16()
    ms = time_ms(lambda: kernels.swiglu_bwd(da, gu))
    emit(kernel="swiglu_bwd", T=T, F=Fh, ms=round(ms, 4), gbs=round(5 * T * Fh * 2 / ms / 1e6, 1))
    logits = torch.randn(T, V, device="cuda").bfloat16()
    labels = torch.randint(0, V, (T,), device="cuda")
    ms = time_ms(lambda: kernels.cross_entropy_(logits, labels, 1.0), iters=5)
    emit(kernel="cross_entropy", T=T, V=V, ms=round(ms, 4), gbs=round(3 * T * V * 2 / ms / 1e6, 1))
    del logits
    n = 1 << 28
    p = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    g = torch.zeros(n, device="cuda", dtype=torch.float32)
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    ms = time_ms(lambda: kernels.adamw_(p, g, m, v, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=1),
                 iters=5)
    emit(kernel="adamw", n=n, ms=round(ms, 4), gbs=round(n * (2 + 2 + 4 + 16) / ms / 1e6, 1))
    _lib.check_status("elementwise")


def bench_fp8(quick: bool) -> None:
    """Per-tensor FP8 GEMM (e4m3 x e4m3, e5m2 x e4m3) and its quantiser."""
    from ..ops import fp8
    shapes = [(M, N, K, tag) for (M, N, K, a_mn, b_mn, tag) in GEMM_SHAPES if not a_mn and not b_mn]
    for M, N, K, tag in (shapes[:3] if quick else shapes):
        a = torch.randn(M, K, device="cuda").bfloat16()
        b = torch.randn(N, K, device="cuda").bfloat16()
        for fa in ("e4m3", "e5m2"):
            sa, sb = fp8.DelayedScale(fa, "cuda"), fp8.DelayedScale("e4m3", "cuda")
            sa.prepare(a, 0)
            sb.prepare(b, 0)
            ms_q = time_ms(lambda: fp8.quantize(a, sa, want_row=True, want_col=True))
            a_op, _ = fp8.quantize(a, sa)
            b_op, _ = fp8.quantize(b, sb)
            out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            ms = time_ms(lambda: fp8.gemm(a_op, b_op, out=out))
            emit(kernel="gemm_fp8", tag=tag, a_fmt=fa, M=M, N=N, K=K, ms=round(ms, 4), tflops=round(2.0 * M * N * K / ms / 1e9, 1),
                 quant_dual_ms=round(ms_q, 4), quant_gbs=round(M * K * 4.0 / ms_q / 1e6, 1))
        _lib.check_status(tag)
        del a, b


def bench_grouped(quick: bool) -> None:
    """Grouped (per-expert) GEMMs of the GPT-OSS MoE layer: 32 experts, hidden 2880, top-4."""
    from ..ops import moe_ops as M
    T, E, k, D, Fh = (8192 if quick else 32768), 32, 4, 2880, 2880
    logits = torch.randn(T, E, device="cuda")
    idx, w, cnt = M.router_topk(logits, k)
    seg, te, dest, rows = M.plan(idx, cnt, E)
    x = torch.randn(T, D, device="cuda").bfloat16()
    w1 = (torch.randn(E, 2 * Fh, D, device="cuda") * 0.02).bfloat16()
    xp = M.permute_rows(x, dest, k, rows)
    ms = time_ms(lambda: M.grouped_rows(xp, w1, te, seg))
    emit(kernel="gemm_grouped fc1", T=T, pairs=T * k, E=E, D=D, N=2 * Fh, ms=round(ms, 4),
         tflops=round(2.0 * T * k * D * 2 * Fh / ms / 1e9, 1))
    ms_p = time_ms(lambda: M.permute_rows(x, dest, k, rows))
    emit(kernel="permute_rows", T=T, k=k, D=D, ms=round(ms_p, 4), gbs=round(T * D * 2 * (1 + k) / ms_p / 1e6, 1))
    _lib.check_status("grouped")
    # the same layer on block-scaled operands (segments padded to 256 rows)
    from ..ops import mxfp8
    w2 = (torch.randn(E, D, Fh, device="cuda") * 0.02).bfloat16()
    seg2, te2, dest2, rows2 = M.plan(idx, cnt, E, pad=M.PAD_MX)
    xp2 = M.permute_rows(x, dest2, k, rows2)
    fl = 2.0 * T * k * D * 2 * Fh
    ms_q = time_ms(lambda: mxfp8.quantize(xp2, row_tile=128, col_tile=M.grouped_bn(D)))
    a_op, at_op = mxfp8.quantize(xp2, row_tile=128, col_tile=M.grouped_bn(D))
    b_op = M._stacked_weight_op(w1, False)
    ms = time_ms(lambda: M.grouped_rows_mx(a_op, b_op, te2, E))
    emit(kernel="gemm_grouped_mx fc1", T=T, pairs=T * k, rows=rows2, E=E, D=D, N=2 * Fh, ms=round(ms, 4),
         tflops=round(fl / ms / 1e9, 1), quant_rows_ms=round(ms_q, 4))
    gu = M.grouped_rows_mx(a_op, b_op, te2, E)
    _, gt_op = mxfp8.quantize(gu, col_tile=128)
    acc = torch.zeros(E, 2 * Fh, D, device="cuda")
    ms = time_ms(lambda: M.grouped_wgrad_mx(gt_op, at_op, seg2, E, acc))
    emit(kernel="gemm_grouped_mx wgrad fc1 (fp32 accumulate)", T=T, E=E, M=2 * Fh, N=D, ms=round(ms, 4),
         tflops=round(fl / ms / 1e9, 1), out_gbs=round(E * 2 * Fh * D * 8 / ms / 1e6, 1))
    xg = x.clone().requires_grad_()
    p1, p2 = w1.clone().requires_grad_(), w2.clone().requires_grad_()
    p1.main_grad, p2.main_grad = torch.zeros_like(p1, dtype=torch.float32), torch.zeros_like(p2, dtype=torch.float32)
    for prec in ("bf16", "mxfp8"):
        def step():
            y = M.moe_experts(xg, idx, w, cnt, p1, p2, prec)
            y.backward(y.detach())
            p1.grad = p2.grad = xg.grad = None
        ms = time_ms(step)
        emit(kernel=f"moe_experts fwd+bwd ({prec})", T=T, E=E, k=k, D=D, F=Fh, ms=round(ms, 4),
             tflops=round(3 * 3 * fl / 2 / ms / 1e9, 1))
    _lib.check_status("grouped mx")


def bench_hstu(quick: bool) -> None:
    """Jagged pointwise-SiLU attention at the HSTU benchmark shape: log-normal lengths, 4 heads of 128."""
    from ..ops.hstu_ops import hstu_attention
    g = torch.Generator().manual_seed(0)
    B = 32 if quick else 128
    lens = torch.exp(torch.randn(B, generator=g) + math.log(512)).clamp(16, 4095).long() + 1
    offs = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)]).to(torch.int32).cuda()
    L, H, D, N = int(lens.sum()), 4, 128, 4096
    q, k, v = (torch.randn(L, H, D, device="cuda").bfloat16().requires_grad_(True) for _ in range(3))
    nt = torch.ones(B, dtype=torch.int32, device="cuda")
    pairs = float((lens.double() ** 2).sum()) / 2
    ms_f = time_ms(lambda: hstu_attention(q, k, v, offs, N, D ** -0.5, nt, 0))
    out = hstu_attention(q, k, v, offs, N, D ** -0.5, nt, 0)
    do = torch.randn_like(out)

    def bwd():
        q.grad = k.grad = v.grad = None
        out.backward(do, retain_graph=True)
    ms_b = time_ms(bwd)
    emit(kernel="hstu_attention", B=B, tokens=L, H=H, D=D, fwd_ms=round(ms_f, 4), fwd_tflops=round(4.0 * H * pairs * D / ms_f / 1e9, 1),
         bwd_ms=round(ms_b, 4), bwd_tflops=round(10.0 * H * pairs * D / ms_b / 1e9, 1))

    class _Owner:                     # keeps the delayed-scaling states of Q, K, V between calls, like a layer does
        pass
    own = _Owner()
    with torch.no_grad():
        ms_8 = time_ms(lambda: hstu_attention(q, k, v, offs, N, D ** -0.5, nt, 0, precision="fp8", owner=own))
    emit(kernel="hstu_attention fp8 forward (3 quantise launches included)", B=B, tokens=L, H=H, D=D, fwd_ms=round(ms_8, 4),
         fwd_tflops=round(4.0 * H * pairs * D / ms_8 / 1e9, 1))
    _lib.check_status("hstu")


def bench_glue(quick: bool) -> None:
    """MMDiT glue kernels at the FLUX shape: 32 samples x 512 tokens x 3072."""
    from ..ops import functional as F
    B, S, D = (8 if quick else 32), 512, 3072
    x = torch.randn(B * S, D, device="cuda").bfloat16().requires_grad_(True)
    mod = torch.randn(B, 3 * D, device="cuda").bfloat16()
    shift, scale, gate = mod.chunk(3, dim=-1)
    ms = time_ms(lambda: F.ln_modulate(x, shift, scale, B, 1e-6))
    emit(kernel="ln_modulate_fwd", T=B * S, D=D, ms=round(ms, 4), gbs=round(2 * B * S * D * 2 / ms / 1e6, 1))
    y = torch.randn(B * S, D, device="cuda").bfloat16()
    ms = time_ms(lambda: F.gate_residual(x, y, gate, B))
    emit(kernel="gate_residual_fwd", T=B * S, D=D, ms=round(ms, 4), gbs=round(3 * B * S * D * 2 / ms / 1e6, 1))
    _lib.check_status("glue")


def bench_sparse(quick: bool) -> None:
    """Sort / unique / segment reduction of the embedding path at the HSTU step size."""
    from ..ops import sort
    n, rows, D = (200_000 if quick else 2_000_000), 400_000_000, 256
    u = torch.rand(n, device="cuda")
    ids = (torch.exp(u * math.log(rows)).long() - 1).clamp(0, rows - 1)        # Zipf-like skew
    ms = time_ms(lambda: sort.sort_unique(ids, sort.key_bits_for(rows)))
    s = sort.sort_unique(ids, sort.key_bits_for(rows))
    g = torch.randn(n, D, device="cuda").bfloat16()
    ms_s = time_ms(lambda: sort.segment_sum(g, s, torch.bfloat16))
    emit(kernel="sort_unique", n=n, key_bits=sort.key_bits_for(rows), ms=round(ms, 4), mkeys_per_s=round(n / ms / 1e3, 1),
         unique=s.n_unique())
    emit(kernel="segment_sum_gather", n=n, D=D, ms=round(ms_s, 4), gbs=round(n * D * 2 * 1.5 / ms_s / 1e6, 1))
    _lib.check_status("sparse")


def bench_comm(quick: bool) -> None:
    """The peer-memory kernels with every "peer" a buffer of THIS GPU (world 8 emulated): the same instruction
    streams as on NVLink, so launch geometry, register use and memory-side behaviour can be profiled on one GPU;
    the bytes that would cross NVLink are reported next to the time.  None of these kernels waits for another rank."""
    import ctypes
    from ..ops import moe_ops as M
    W = 8
    arr = lambda ts: (ctypes.c_ulonglong * len(ts))(*[t.data_ptr() for t in ts])
    # ZeRO step: reduce-scatter of fp32 gradients by peer loads, AdamW + all-gather by peer stores
    n_total = (16 if quick else 64) * 1024 * 1024
    n = n_total // W
    grads = [torch.randn(n_total, device="cuda") for _ in range(W)]
    out = torch.empty(n, device="cuda")
    part = torch.zeros(_lib.load().b200_zero_grid(), device="cuda")
    ms = time_ms(lambda: _lib.call("b200_zero_reduce_scatter", arr(grads), W, 1, n, n, 1.0 / W, _lib.ptr(out), _lib.ptr(part),
                                   _lib.stream_ptr()))
    emit(kernel="zero_reduce_scatter (8 emulated ranks)", shard_elems=n, ms=round(ms, 4), read_gbs=round(W * n * 4 / ms / 1e6, 1),
         nvlink_mb=round((W - 1) * n * 4 / 1e6, 1))
    del grads
    params = [torch.zeros(n_total, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    m, v, master = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda"), torch.randn(n, device="cuda")
    sumsq = torch.ones(1, device="cuda")
    ms = time_ms(lambda: _lib.call("b200_zero_adamw_all_gather", arr(params), W, 1, n, n, _lib.ptr(out), _lib.ptr(m), _lib.ptr(v),
                                   _lib.ptr(master), 1e-3, 0.9, 0.95, 1e-8, 0.1, 1, 1.0, _lib.ptr(sumsq), 1.0, 0, _lib.stream_ptr()))
    emit(kernel="zero_adamw_all_gather (8 emulated ranks)", shard_elems=n, ms=round(ms, 4),
         local_gbs=round(n * (4 * 4 + 3 * 4) / ms / 1e6, 1), nvlink_mb=round((W - 1) * n * 2 / 1e6, 1))
    del params, m, v, master
    # expert dispatch: scatter rows into the owners' slabs, gather rows back
    T, k, D = (4096 if quick else 8192), 4, 2880
    rows = T * k
    cap = 2 * rows
    slabs = [torch.zeros(cap, D, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    src = torch.randn(rows, D, device="cuda").bfloat16()
    dst_rank = torch.randint(0, W, (rows,), device="cuda", dtype=torch.int32)
    dst_row = torch.randperm(cap, device="cuda")[:rows].to(torch.int32)
    dropped = torch.zeros(1, dtype=torch.int32, device="cuda")
    ms = time_ms(lambda: _lib.call("b200_scatter_rows_to_peers", _lib.ptr(src), None, _lib.ptr(dst_rank), _lib.ptr(dst_row), rows, D,
                                   arr(slabs), W, cap, _lib.ptr(dropped), _lib.stream_ptr()))
    emit(kernel="scatter_rows_to_peers (8 emulated ranks)", rows=rows, D=D, ms=round(ms, 4), gbs=round(2 * rows * D * 2 / ms / 1e6, 1),
         nvlink_mb=round((W - 1) / W * rows * D * 2 / 1e6, 1))
    back = torch.empty(rows, D, device="cuda", dtype=torch.bfloat16)
    ms = time_ms(lambda: _lib.call("b200_gather_rows_from_peers", arr(slabs), _lib.ptr(dst_rank), _lib.ptr(dst_row), rows, D,
                                   _lib.ptr(back), W, cap, _lib.stream_ptr()))
    emit(kernel="gather_rows_from_peers (8 emulated ranks)", rows=rows, D=D, ms=round(ms, 4), gbs=round(2 * rows * D * 2 / ms / 1e6, 1))
    del slabs
    # routing tables of the dispatch in one kernel
    E, L = 32, 4
    allc = torch.randint(900, 1200, (W, E), device="cuda", dtype=torch.int32)
    seg = torch.cat([torch.zeros(1, dtype=torch.int32, device="cuda"), allc[1].cumsum(0).to(torch.int32)])
    npairs = int(seg[-1])
    outs = [torch.empty(npairs, dtype=torch.int32, device="cuda") for _ in range(2)]
    seg2, cnt2 = torch.empty(L + 1, dtype=torch.int32, device="cuda"), torch.empty(L, dtype=torch.int32, device="cuda")
    capr = 2 * npairs // 256 * 256
    te = torch.empty(capr // 256, dtype=torch.int32, device="cuda")
    ms = time_ms(lambda: _lib.call("b200_ep_route", _lib.ptr(allc), _lib.ptr(seg), W, E, 1, 256, capr, npairs, _lib.ptr(outs[0]),
                                   _lib.ptr(outs[1]), _lib.ptr(seg2), _lib.ptr(cnt2), _lib.ptr(te), _lib.stream_ptr()))
    emit(kernel="ep_route", pairs=npairs, experts=E, ms=round(ms, 4))
    # all-gather -> GEMM with two emulated ranks (pull mode: the copy CTAs of the launch fetch the other block)
    rows_per, K, N = 2048, (4096 if quick else 8192), 3584
    x = (torch.randn(2 * rows_per, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
    bufs = [x.clone(), x.clone()]
    o = torch.empty(2 * rows_per, N, device="cuda", dtype=torch.bfloat16)
    flags = torch.zeros(32, dtype=torch.int32, device="cuda")

    def ag():
        flags.zero_()
        _lib.call("b200_gemm_tp_gather", _lib.ptr(bufs[0]), _lib.ptr(w), _lib.ptr(o), 2 * rows_per, N, K, K, K, N, 0, 0, 0, 0, 1.0, 1,
                  arr(bufs), 2, 0, _lib.ptr(bufs[0]), rows_per * K * 2, rows_per, _lib.ptr(flags), 8, 0, None, _lib.stream_ptr())
    ms = time_ms(ag)
    emit(kernel="gemm_tp all-gather -> GEMM (2 emulated ranks, pull)", M=2 * rows_per, N=N, K=K, ms=round(ms, 4),
         tflops=round(2.0 * 2 * rows_per * N * K / ms / 1e9, 1), pulled_mb=round(rows_per * K * 2 / 1e6, 1))
    stage = torch.empty(2 * rows_per, N, device="cuda", dtype=torch.bfloat16)
    rs_flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    work = torch.zeros(1, dtype=torch.int32, device="cuda")
    o2 = torch.empty(2 * rows_per, N, device="cuda", dtype=torch.bfloat16)

    def rs():
        rs_flags.zero_(); work.zero_()
        _lib.call("b200_gemm_tp_rs", _lib.ptr(x), _lib.ptr(w), 2 * rows_per, N, K, K, K, 0, 0, 1.0, arr([stage]), arr([rs_flags]), 1, 0,
                  _lib.ptr(work), _lib.ptr(o2), N, None, 0, 8, _lib.stream_ptr())
    ms = time_ms(rs)
    emit(kernel="gemm_tp GEMM -> reduce-scatter (world 1: staging + reduce queue)", M=2 * rows_per, N=N, K=K, ms=round(ms, 4),
         tflops=round(2.0 * 2 * rows_per * N * K / ms / 1e9, 1))
    _lib.check_status("comm")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("what", nargs="*", default=["gemm", "attention", "elementwise"])
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--iters", type=int, default=10, help="timed launches per measurement")
    ap.add_argument("--warmup", type=int, default=3, help="untimed launches per measurement")
    args = ap.parse_args(argv)
    global ITERS, WARMUP
    ITERS, WARMUP = max(args.iters, 1), max(args.warmup, 0)
    if not torch.cuda.is_available():
        print("microbench needs a CUDA device", file=sys.stderr)
        return 1
    for w in args.what:
        {"gemm": bench_gemm, "mxfp8": bench_mxfp8, "fp8": bench_fp8, "attention": bench_attention, "elementwise": bench_elementwise,
         "grouped": bench_grouped, "hstu": bench_hstu, "glue": bench_glue, "sparse": bench_sparse, "comm": bench_comm}[w](args.quick)
    return 0


if __name__ == "__main__":
    sys.exit(main())
