"""Kernels at the shapes of the benchmark configurations (the small-shape files test layouts and edge
cases; these test the long contraction, the wide vocabulary, the 8192-token sequence and the 2880-wide
experts), compared tile by tile."""
import math

import pytest
import torch

from mlperf_training_b200.ops import _lib, kernels, moe_ops as M, mxfp8

from ._tol import assert_tiles_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M_,N,K", [(2048, 4096, 14336), (2048, 128256, 4096), (4096, 28672, 4096)])
def test_mxfp8_gemm_bench_shapes(M_, N, K):
    torch.manual_seed(N)
    a = torch.randn(M_, K, device="cuda").bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    a_op, _ = mxfp8.quantize(a, row_tile=mxfp8.A_TILE)
    b_op, _ = mxfp8.quantize(b, row_tile=mxfp8.b_tile(N))
    d = mxfp8.gemm(a_op, b_op)
    torch.cuda.synchronize()
    _lib.check_status("mxfp8 bench shape")
    ref = torch.empty(M_, N, device="cuda")
    bd = mxfp8.dequantize(b_op)
    ad = mxfp8.dequantize(a_op)
    for n0 in range(0, N, 16384):                              # fp32 reference in column chunks
        ref[:, n0:n0 + 16384] = ad @ bd[n0:n0 + 16384].t()
    assert_tiles_close(d, ref, rel=6e-3, what=f"mxfp8 {M_}x{N}x{K}")
    acc = torch.zeros(M_, N, device="cuda")
    mxfp8.gemm(a_op, b_op, out=acc, accumulate=True)
    torch.cuda.synchronize()
    assert_tiles_close(acc, ref, rel=1e-4, what="fp32 accumulate")


@pytest.mark.parametrize("M_,N,K,a_mn,b_mn", [(8192, 6144, 4096, False, False), (4096, 14336, 8192, True, True),
                                              (8192, 4096, 14336, False, True)])
def test_bf16_gemm_bench_shapes(M_, N, K, a_mn, b_mn):
    torch.manual_seed(K)
    a = torch.randn((K, M_) if a_mn else (M_, K), device="cuda").bfloat16()
    b = (torch.randn((K, N) if b_mn else (N, K), device="cuda") * 0.05).bfloat16()
    d = kernels.gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn, out_dtype=torch.float32)
    torch.cuda.synchronize()
    _lib.check_status("bf16 bench shape")
    ref = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
    assert_tiles_close(d, ref, rel=1e-4, what=f"bf16 {M_}x{N}x{K}")


def _attention_reference_chunked(q, k, v, scale, chunk=1024):
    """fp32 causal GQA attention of ``[1, S, H, D]`` tensors computed in query chunks."""
    S, Hq, D = q.shape[1], q.shape[2], q.shape[3]
    g = Hq // k.shape[2]
    kf = k[0].float().repeat_interleave(g, 1).transpose(0, 1)      # [Hq, S, D]
    vf = v[0].float().repeat_interleave(g, 1).transpose(0, 1)
    out = torch.empty(S, Hq, D, device=q.device)
    pos = torch.arange(S, device=q.device)
    for s0 in range(0, S, chunk):
        qc = q[0, s0:s0 + chunk].float().transpose(0, 1)           # [Hq, c, D]
        sc = torch.matmul(qc, kf.transpose(1, 2)) * scale
        sc = sc.masked_fill(pos[None, None, :] > pos[s0:s0 + chunk][None, :, None], float("-inf"))
        out[s0:s0 + chunk] = torch.matmul(torch.softmax(sc, -1), vf).transpose(0, 1)
    return out[None]


def test_attention_at_sequence_8192():
    torch.manual_seed(0)
    B, S, Hq, Hkv, D = 1, 8192, 8, 2, 128
    q = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    do = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    scale = 1 / math.sqrt(D)
    o, lse = kernels.attention_fwd(q, k, v, scale=scale, causal=True)
    dq, dk, dv, _ = kernels.attention_bwd(do, q, k, v, o, lse, scale=scale, causal=True)
    torch.cuda.synchronize()
    _lib.check_status("attention S=8192")
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    ref = _attention_reference_chunked(qf, kf, vf, scale)
    ref.backward(do.float())
    assert_tiles_close(o[0].reshape(S, -1), ref[0].detach().reshape(S, -1), rel=2e-2, cos=0.9995, what="o")
    assert_tiles_close(dq[0].reshape(S, -1), qf.grad[0].reshape(S, -1), rel=4e-2, cos=0.999, what="dq")
    assert_tiles_close(dk[0].reshape(S, -1), kf.grad[0].reshape(S, -1), rel=4e-2, cos=0.999, what="dk")
    assert_tiles_close(dv[0].reshape(S, -1), vf.grad[0].reshape(S, -1), rel=4e-2, cos=0.999, what="dv")


def test_grouped_gemm_at_gpt_oss_expert_width():
    torch.manual_seed(1)
    T, E, k, D, Fh = 8192, 32, 4, 2880, 2880
    logits = torch.randn(T, E, device="cuda")
    idx, w, cnt = M.router_topk(logits, k)
    seg, te, dest, rows = M.plan(idx, cnt, E)
    x = (torch.randn(T, D, device="cuda") * 0.5).bfloat16()
    w1 = (torch.randn(E, 2 * Fh, D, device="cuda") * 0.02).bfloat16()
    xp = M.permute_rows(x, dest, k, rows)
    out = M.grouped_rows(xp, w1, te, seg)
    torch.cuda.synchronize()
    _lib.check_status("grouped 2880")
    te_h, seg_h = te.cpu().tolist(), seg.cpu().tolist()
    for t, e in enumerate(te_h):
        if e < 0 or t % 7:                                         # every 7th live tile against the expert's fp32 product
            continue
        r0 = t * M.PAD
        ref = xp[r0:r0 + M.PAD].float() @ w1[e].float().t()
        assert_tiles_close(out[r0:r0 + M.PAD], ref, rel=8e-3, what=f"grouped tile {t} expert {e}")
