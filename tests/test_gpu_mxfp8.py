"""MXFP8 quantiser and block-scaled tcgen05 GEMM against the eager emulation (bit-exact codes and
scales; GEMM against an fp32 matmul of the dequantised operands)."""
import pytest
import torch

from mlperf_training_b200.ops import _lib, mxfp8

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("R,C", [(128, 128), (256, 384), (896, 512)])
def test_quantize_matches_emulation(R, C):
    torch.manual_seed(R + C)
    x = (torch.randn(R, C) * torch.exp(torch.randn(R, 1) * 2)).bfloat16()
    x[3, 32:64] = 0  # an all-zero block
    x[5, 0] = 448.0 * 4  # amax exactly on a power-of-two boundary
    for row_tile, col_tile in ((128, 224), (224, 128)):
        r_c, c_c = mxfp8.quantize(x, row_tile=row_tile, col_tile=col_tile)
        r_g, c_g = mxfp8.quantize(x.cuda(), row_tile=row_tile, col_tile=col_tile)
        torch.cuda.synchronize()
        for cpu, gpu, what in ((r_c, r_g, "row"), (c_c, c_g, "col")):
            assert torch.equal(mxfp8.sf_plain(gpu).cpu(), cpu.sf), f"{what} scales"
            assert torch.equal(gpu.q.cpu(), cpu.q), f"{what} codes"
        # quantisation error is bounded by the e4m3 step
        err = (mxfp8.dequantize(r_g).cpu() - x.float()).abs()
        assert (err <= x.float().abs().view(R, C // 32, 32).amax(-1, keepdim=True).expand(-1, -1, 32).reshape(R, C) * 0.07 + 1e-30).all()


@pytest.mark.parametrize("R,C", [(256, 160), (384, 960), (2048, 2880)])
def test_quantize_partial_column_tile(R, C):
    """Widths that are multiples of 32 but not of 128 (the last 128-column tile is partial)."""
    torch.manual_seed(R + C)
    x = (torch.randn(R, C) * torch.exp(torch.randn(R, 1))).bfloat16()
    r_c, c_c = mxfp8.quantize(x, row_tile=128, col_tile=192)
    r_g, c_g = mxfp8.quantize(x.cuda(), row_tile=128, col_tile=192)
    torch.cuda.synchronize()
    _lib.check_status("quant partial")
    for cpu, gpu, what in ((r_c, r_g, "row"), (c_c, c_g, "col")):
        assert torch.equal(mxfp8.sf_plain(gpu).cpu(), cpu.sf), f"{what} scales"
        assert torch.equal(gpu.q.cpu(), cpu.q), f"{what} codes"
    gu = (torch.randn(R, 2 * C) * 2).bfloat16()
    a_c, at_c = mxfp8.quantize_swiglu(gu, row_tile=128, col_tile=192)
    a_g, at_g = mxfp8.quantize_swiglu(gu.cuda(), row_tile=128, col_tile=192)
    ref = mxfp8.dequantize(a_c)
    assert (mxfp8.dequantize(a_g).cpu() - ref).abs().max() <= 0.13 * ref.abs().max()      # SwiGLU rounding may flip a code
    assert (mxfp8.dequantize(at_g).cpu() - mxfp8.dequantize(at_c)).abs().max() <= 0.13 * ref.abs().max()


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 224, 256), (384, 448, 512), (512, 1000, 384),
                                   (1024, 4096, 1024), (136, 72, 128)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_mxfp8(M, N, K, out_dtype):
    torch.manual_seed(M + N + K)
    Mp, Np = (M + 127) // 128 * 128, (N + 127) // 128 * 128
    a = torch.randn(Mp, K, device="cuda").bfloat16()
    b = torch.randn(Np, K, device="cuda").bfloat16()
    a_op, _ = mxfp8.quantize(a, row_tile=mxfp8.A_TILE)
    b_op, _ = mxfp8.quantize(b, row_tile=mxfp8.b_tile(Np))
    d = mxfp8.gemm(a_op, b_op, out_dtype=out_dtype)
    torch.cuda.synchronize()
    _lib.check_status("gemm_mxfp8")
    ref = mxfp8.dequantize(a_op) @ mxfp8.dequantize(b_op).t()
    err = (d.float() - ref).abs().max().item()
    tol = (2e-2 if out_dtype == torch.bfloat16 else 1e-3) * ref.abs().max().item()
    assert err <= tol, f"err {err} tol {tol}"
    # and the quantised product is close to the bf16 product
    full = a.float() @ b.float().t()
    rel = (ref - full).norm() / full.norm()
    assert rel < 0.06


def test_gemm_mxfp8_epilogues():
    torch.manual_seed(0)
    M, N, K = 256, 512, 256
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    a_op, _ = mxfp8.quantize(a, row_tile=mxfp8.A_TILE)
    b_op, _ = mxfp8.quantize(b, row_tile=mxfp8.b_tile(N))
    ref = mxfp8.dequantize(a_op) @ mxfp8.dequantize(b_op).t()
    res = torch.randn(M, N, device="cuda").bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    d = mxfp8.gemm(a_op, b_op, residual=res, bias=bias, alpha=0.5)
    acc = torch.ones(M, N, device="cuda")
    mxfp8.gemm(a_op, b_op, out=acc, accumulate=True)
    mxfp8.gemm(a_op, b_op, out=acc, accumulate=True)
    torch.cuda.synchronize()
    sc = ref.abs().max().item()
    assert (d.float() - (0.5 * ref + res.float() + bias.float())).abs().max().item() < 2e-2 * sc
    assert (acc - (2 * ref + 1)).abs().max().item() < 2e-3 * sc
    _lib.check_status("gemm_mxfp8 epilogues")


def test_fused_mlp_matches_unfused_mxfp8_path():
    """The fused unit (quantisation folded into SwiGLU / dSwiGLU) computes exactly what the separate
    norm_linear + swiglu_linear MXFP8 path computes."""
    import torch
    from mlperf_training_b200.ops import functional as F
    torch.manual_seed(0)
    T, D, Fh = 512, 256, 512
    h0 = torch.randn(T, D, device="cuda").bfloat16()
    nw0 = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16()
    w1_0 = (torch.randn(2 * Fh, D, device="cuda") * 0.05).bfloat16()
    w2_0 = (torch.randn(D, Fh, device="cuda") * 0.05).bfloat16()
    dy = torch.randn(T, D, device="cuda").bfloat16()
    outs = []
    for fused in (False, True):
        h, nw, w1, w2 = (t.clone().requires_grad_(True) for t in (h0, nw0, w1_0, w2_0))
        assert F.fused_mlp_eligible(h, w1, w2)
        if fused:
            y = F.fused_mlp(h, nw, w1, w2, 1e-5)
        else:
            gu = F.norm_linear(h, nw, w1, eps=1e-5, precision="mxfp8")
            y = F.swiglu_linear(gu, w2, residual=h, precision="mxfp8")
        y.backward(dy)
        outs.append([t.detach().float() for t in (y, h.grad, nw.grad, w1.grad, w2.grad)])
    torch.cuda.synchronize()
    for name, a, b in zip(("y", "dh", "dnorm", "dw1", "dw2"), outs[0], outs[1]):
        if name == "dh":
            # the fused unit adds the residual gradient inside the norm backward (one rounding instead of two)
            assert (a - b).abs().max().item() <= 2.0 ** -6 * max(1.0, b.abs().max().item()), name
        else:
            assert torch.equal(a, b), (name, (a - b).abs().max().item())


@pytest.mark.parametrize("fmt", ["e2m1", "e2m3", "e3m2"])
def test_narrow_element_formats_match_the_cpu_oracle(fmt):
    """Operands rounded to a 4- / 6-bit element grid and carried as e4m3 codes: the same codes and scales as the CPU
    routine, and the block-scaled GEMM multiplies them like the dequantised matrices."""
    torch.manual_seed(0)
    x = (torch.randn(256, 384) * torch.logspace(-2, 1, 384)[None, :]).bfloat16()
    w = (torch.randn(256, 384) * 0.05).bfloat16()
    a_c = mxfp8.quantize(x, row_tile=mxfp8.A_TILE, fmt=fmt)[0]
    a_g = mxfp8.quantize(x.cuda(), row_tile=mxfp8.A_TILE, fmt=fmt)[0]
    assert torch.equal(a_g.q.cpu(), a_c.q) and torch.equal(mxfp8.sf_plain(a_g).cpu(), a_c.sf)
    bt = mxfp8.b_tile(256)
    b_c = mxfp8.quantize(w, row_tile=bt, fmt=fmt)[0]
    b_g = mxfp8.quantize(w.cuda(), row_tile=bt, fmt=fmt)[0]
    y_g = mxfp8.gemm(a_g, b_g, out_dtype=torch.float32)
    y_c = mxfp8.gemm(a_c, b_c, out_dtype=torch.float32)
    assert (y_g.cpu() - y_c).abs().max() <= 1e-3 * y_c.abs().max()
    _, col_g = mxfp8.quantize(x.cuda(), col_tile=bt, fmt="e4m3", col_fmt=fmt)
    _, col_c = mxfp8.quantize(x, col_tile=bt, fmt="e4m3", col_fmt=fmt)
    assert torch.equal(col_g.q.cpu(), col_c.q) and torch.equal(mxfp8.sf_plain(col_g).cpu(), col_c.sf)


@pytest.mark.parametrize("recipe", ["mxfp4", "a6w4"])
def test_narrow_recipes_through_the_linear_triple(recipe):
    from mlperf_training_b200.ops import functional as F
    torch.manual_seed(1)
    x = torch.randn(256, 256).bfloat16()
    w = (torch.randn(384, 256) * 0.05).bfloat16()
    g = torch.randn(256, 384).bfloat16()
    y_c = F.linear(x, w, None, None, recipe)
    xg, wg = x.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
    y_g = F.linear(xg, wg, None, None, recipe)
    assert (y_g.float().cpu() - y_c.float()).abs().max() <= 2e-2 * y_c.float().abs().max()      # same operands, bf16 output
    y_g.backward(g.cuda())
    ref_dx, ref_dw = g.float() @ w.float(), g.float().t() @ x.float()
    rel = lambda a, b: float((a.float().cpu() - b).norm() / b.norm())
    assert rel(xg.grad, ref_dx) < 0.3 and rel(wg.grad, ref_dw) < 0.3        # stochastic 4-bit gradients: close, not equal
    _lib.check_status("narrow recipes")
