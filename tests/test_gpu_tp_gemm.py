"""Tensor-parallel GEMM kernels on one GPU: world 1 (all three modes), and the all-gather modes with
two emulated ranks whose launches run one after the other (a gather launch waits only on its own
copy CTAs, never on another rank's kernel)."""
import ctypes

import pytest
import torch

from mlperf_training_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _arr(ptrs):
    return (ctypes.c_ulonglong * len(ptrs))(*ptrs)


def _gather_call(a, b, out, M, N, K, a_mn, b_mn, mode, bufs, rank, full, rows_per, chunk_bytes, accumulate=False):
    W = len(bufs)
    flags = torch.zeros(32, dtype=torch.int32, device="cuda")
    _lib.call("b200_gemm_tp_gather", _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), M, N, K, a.stride(0), b.stride(0),
              out.stride(0), a_mn, b_mn, int(out.dtype == torch.float32), int(accumulate), 1.0, mode,
              _arr([t.data_ptr() for t in bufs]), W, rank, _lib.ptr(full), chunk_bytes, rows_per, _lib.ptr(flags), 4,
              0, None, _lib.stream_ptr())        # pull mode: the launch depends on no other rank's kernel
    torch.cuda.synchronize()
    _lib.check_status("gemm_tp_gather")


@pytest.mark.parametrize("W", [1, 2, 4])
@pytest.mark.parametrize("N", [384, 128])
def test_all_gather_gemm_rows(W, N):
    torch.manual_seed(W * 10 + N)
    rows_per, K = 256, 320
    T = W * rows_per
    x = (torch.randn(T, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    want = x.float() @ w.float().t()
    bufs = []
    for r in range(W):                                    # each rank's buffer holds only its own row block
        buf = torch.full((T, K), float("nan"), device="cuda").bfloat16()
        buf[r * rows_per:(r + 1) * rows_per] = x[r * rows_per:(r + 1) * rows_per]
        bufs.append(buf)
    for r in range(W):
        out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
        _gather_call(bufs[r], w, out, T, N, K, 0, 0, 1, bufs, r, bufs[r], rows_per, rows_per * K * 2)
        assert torch.equal(bufs[r], x), f"rank {r}: gathered operand differs"
        err = (out.float() - want).abs().max().item()
        assert err < 2e-2 * want.abs().max().item(), (r, err)


@pytest.mark.parametrize("W", [1, 2])
def test_all_gather_gemm_reduction_dim(W):
    """wgrad: dW[N, K] = dy[T, N]^T x_full[T, K], x gathered along T (the reduction)."""
    torch.manual_seed(5 + W)
    rows_per, K, N = 192, 256, 320
    T = W * rows_per
    x = (torch.randn(T, K, device="cuda") * 0.5).bfloat16()
    dy = (torch.randn(T, N, device="cuda") * 0.5).bfloat16()
    want = dy.float().t() @ x.float()
    bufs = []
    for r in range(W):
        buf = torch.full((T, K), float("nan"), device="cuda").bfloat16()
        buf[r * rows_per:(r + 1) * rows_per] = x[r * rows_per:(r + 1) * rows_per]
        bufs.append(buf)
    for r in range(W):
        acc = torch.ones(N, K, device="cuda", dtype=torch.float32)
        _gather_call(dy, bufs[r], acc, N, K, T, 1, 1, 2, bufs, r, bufs[r], rows_per, rows_per * K * 2, accumulate=True)
        err = (acc - 1.0 - want).abs().max().item()
        assert err < 1e-2 * want.abs().max().item(), (r, err)


@pytest.mark.parametrize("shape", [(256, 384, 320), (1024, 1024, 512)])
@pytest.mark.parametrize("res", [False, True])
def test_gemm_reduce_scatter_world1(shape, res):
    M, N, K = shape
    torch.manual_seed(M + N)
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    resid = torch.randn(M, N, device="cuda").bfloat16() if res else None
    stage = torch.full((M, N), float("nan"), device="cuda").bfloat16()
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    work = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    _lib.call("b200_gemm_tp_rs", _lib.ptr(a), _lib.ptr(b), M, N, K, a.stride(0), b.stride(0), 0, 0, 1.0,
              _arr([stage.data_ptr()]), _arr([flags.data_ptr()]), 1, 0, _lib.ptr(work), _lib.ptr(out), out.stride(0),
              _lib.ptr(resid), 0 if resid is None else resid.stride(0), 4, _lib.stream_ptr())
    torch.cuda.synchronize()
    _lib.check_status("gemm_tp_rs")
    want = (a.float() @ b.float().t()).bfloat16().float()
    if res:
        want = want + resid.float()
    err = (out.float() - want).abs().max().item()
    assert err < 2e-2 * want.abs().max().item(), err
    assert int(work.item()) >= (M // 128) * 64


@pytest.mark.parametrize("W", [1, 2])
@pytest.mark.parametrize("a_fmt", ["e4m3", "e5m2"])
def test_all_gather_gemm_rows_fp8(W, a_fmt):
    """8-bit operands: the gathered blocks are codes, the result is decoded with the two per-tensor factors."""
    from mlperf_training_b200.ops import fp8
    torch.manual_seed(W)
    rows_per, K, N = 256, 384, 384
    T = W * rows_per
    x = (torch.randn(T, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    sx, sw = fp8.DelayedScale(a_fmt, "cuda"), fp8.DelayedScale("e4m3", "cuda")
    sx.prepare(x, 0); sw.prepare(w, 0)
    xq, _ = fp8.quantize(x, sx)
    wq, _ = fp8.quantize(w, sw)
    want = fp8.dequantize(xq) @ fp8.dequantize(wq).t()
    bufs = []
    for r in range(W):
        buf = torch.full((T, K), 0x7f, device="cuda", dtype=torch.uint8)
        buf[r * rows_per:(r + 1) * rows_per] = xq.q[r * rows_per:(r + 1) * rows_per]
        bufs.append(buf)
    for r in range(W):
        out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
        flags = torch.zeros(32, dtype=torch.int32, device="cuda")
        _lib.call("b200_gemm_tp_gather_fp8", _lib.ptr(bufs[r]), _lib.ptr(wq.q), _lib.ptr(out), T, N, K, K, K, N,
                  int(a_fmt == "e5m2"), 0, _lib.ptr(sx.inv_scale), _lib.ptr(sw.inv_scale), 0, 0, 1.0, 1,
                  _arr([t.data_ptr() for t in bufs]), W, r, _lib.ptr(bufs[r]), rows_per * K, rows_per, _lib.ptr(flags), 4, 0,
                  None, _lib.stream_ptr())
        torch.cuda.synchronize()
        _lib.check_status("gemm_tp_gather_fp8")
        assert torch.equal(bufs[r], xq.q), f"rank {r}: gathered codes differ"
        err = (out.float() - want).abs().max().item()
        assert err < 1e-2 * want.abs().max().item(), (r, err)


def test_gemm_reduce_scatter_fp8_world1():
    from mlperf_training_b200.ops import fp8
    torch.manual_seed(9)
    M, N, K = 512, 384, 640
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    sa, sb = fp8.DelayedScale("e5m2", "cuda"), fp8.DelayedScale("e4m3", "cuda")
    sa.prepare(a, 0); sb.prepare(b, 0)
    aq, _ = fp8.quantize(a, sa)
    bq, _ = fp8.quantize(b, sb)
    resid = torch.randn(M, N, device="cuda").bfloat16()
    stage = torch.full((M, N), float("nan"), device="cuda").bfloat16()
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    work = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    _lib.call("b200_gemm_tp_rs_fp8", _lib.ptr(aq.q), _lib.ptr(bq.q), M, N, K, K, K, 1, 0, _lib.ptr(sa.inv_scale),
              _lib.ptr(sb.inv_scale), 1.0, _arr([stage.data_ptr()]), _arr([flags.data_ptr()]), 1, 0, _lib.ptr(work),
              _lib.ptr(out), out.stride(0), _lib.ptr(resid), resid.stride(0), 4, _lib.stream_ptr())
    torch.cuda.synchronize()
    _lib.check_status("gemm_tp_rs_fp8")
    want = (fp8.dequantize(aq) @ fp8.dequantize(bq).t()).bfloat16().float() + resid.float()
    err = (out.float() - want).abs().max().item()
    assert err < 2e-2 * want.abs().max().item(), err


@pytest.mark.parametrize("W", [1, 2])
@pytest.mark.parametrize("fp8_fmt", [None, "e4m3"])
@pytest.mark.parametrize("N", [384, 128])
def test_all_gather_gemm_rows_pair_core(W, fp8_fmt, N):
    """The CTA-pair kernel with copy pairs inside the launch (emulated ranks, pull mode), bf16 and 8-bit operands."""
    from mlperf_training_b200.ops import fp8
    torch.manual_seed(W + N)
    rows_per, K = 512, 640
    T = W * rows_per
    x = (torch.randn(T, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    if fp8_fmt:
        sx, sw = fp8.DelayedScale(fp8_fmt, "cuda"), fp8.DelayedScale("e4m3", "cuda")
        sx.prepare(x, 0); sw.prepare(w, 0)
        xq, _ = fp8.quantize(x, sx)
        wq, _ = fp8.quantize(w, sw)
        src, wt, esz = xq.q, wq.q, 1
        want = fp8.dequantize(xq) @ fp8.dequantize(wq).t()
    else:
        src, wt, esz = x, w, 2
        want = x.float() @ w.float().t()
    bufs = []
    for r in range(W):
        buf = torch.zeros_like(src)
        buf[r * rows_per:(r + 1) * rows_per] = src[r * rows_per:(r + 1) * rows_per]
        bufs.append(buf)
    for r in range(W):
        out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
        flags = torch.zeros(32, dtype=torch.int32, device="cuda")
        _lib.call("b200_gemm_tp_gather_pair", _lib.ptr(bufs[r]), _lib.ptr(wt), _lib.ptr(out), T, N, K, K, K, N,
                  int(bool(fp8_fmt)), 0, 0, _lib.ptr(sx.inv_scale) if fp8_fmt else None, _lib.ptr(sw.inv_scale) if fp8_fmt else None,
                  1.0, _arr([t.data_ptr() for t in bufs]), W, r, _lib.ptr(bufs[r]), rows_per * K * esz, rows_per,
                  _lib.ptr(flags), 4, 0, None, _lib.stream_ptr())
        torch.cuda.synchronize()
        _lib.check_status("gemm_tp_gather_pair")
        assert torch.equal(bufs[r], src), f"rank {r}: gathered operand differs"
        err = (out.float() - want).abs().max().item()
        assert err < 2e-2 * want.abs().max().item(), (r, err)


@pytest.mark.parametrize("shape", [(512, 384, 320), (1024, 128, 512)])
@pytest.mark.parametrize("fp8_on", [False, True])
@pytest.mark.parametrize("res", [False, True])
def test_gemm_reduce_scatter_pair_core_world1(shape, fp8_on, res):
    """GEMM -> reduce-scatter on the CTA-pair core, world 1: tiles through the staging buffer, counters, reduce queue."""
    from mlperf_training_b200.ops import fp8
    M, N, K = shape
    torch.manual_seed(M + N)
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    inv_a = inv_b = None
    if fp8_on:
        K = (K + 127) // 128 * 128
        a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
        b = (torch.randn((N + 127) // 128 * 128, K, device="cuda") * 0.5).bfloat16()
        sa, sb = fp8.DelayedScale("e5m2", "cuda"), fp8.DelayedScale("e4m3", "cuda")
        sa.prepare(a, 0); sb.prepare(b, 0)
        aq, _ = fp8.quantize(a, sa)
        bq, _ = fp8.quantize(b, sb)
        N = b.shape[0]
        want = (fp8.dequantize(aq) @ fp8.dequantize(bq).t()).bfloat16().float()
        A, B, inv_a, inv_b = aq.q, bq.q, sa.inv_scale, sb.inv_scale
    else:
        want = (a.float() @ b.float().t()).bfloat16().float()
        A, B = a, b
    resid = torch.randn(M, N, device="cuda").bfloat16() if res else None
    stage = torch.full((M, N), float("nan"), device="cuda").bfloat16()
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    work = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    _lib.call("b200_gemm_tp_rs_pair", _lib.ptr(A), _lib.ptr(B), M, N, K, K, K, int(fp8_on), int(fp8_on), 0, _lib.ptr(inv_a),
              _lib.ptr(inv_b), 1.0, _arr([stage.data_ptr()]), _arr([flags.data_ptr()]), 1, 0, _lib.ptr(work), _lib.ptr(out),
              out.stride(0), _lib.ptr(resid), 0 if resid is None else resid.stride(0), 4, _lib.stream_ptr())
    torch.cuda.synchronize()
    _lib.check_status("gemm_tp_rs_pair")
    if res:
        want = want + resid.float()
    err = (out.float() - want).abs().max().item()
    assert err < 2e-2 * want.abs().max().item(), err
