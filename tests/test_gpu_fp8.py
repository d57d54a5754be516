"""Per-tensor FP8 quantiser and tcgen05 kind::f8f6f4 GEMM against the eager emulation."""
import pytest
import torch

from mlperf_training_b200.ops import _lib, fp8
from mlperf_training_b200.ops import functional as F

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
def test_quantize_matches_emulation(fmt):
    torch.manual_seed(0)
    x = (torch.randn(384, 256) * 2.5).bfloat16()
    st_c, st_g = fp8.DelayedScale(fmt, "cpu"), fp8.DelayedScale(fmt, "cuda")
    st_c.prepare(x, 0)
    st_g.prepare(x.cuda(), 0)
    rc, cc = fp8.quantize(x, st_c, want_row=True, want_col=True)
    rg, cg = fp8.quantize(x.cuda(), st_g, want_row=True, want_col=True)
    torch.cuda.synchronize()
    assert torch.equal(rg.q.cpu(), rc.q) and torch.equal(cg.q.cpu(), cc.q)
    assert float(st_g.amax.view(torch.float32)) == float(x.abs().max())


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (384, 512, 256), (1024, 4096, 1024), (512, 128, 384)])
@pytest.mark.parametrize("fmts", [("e4m3", "e4m3"), ("e5m2", "e4m3")])
def test_gemm_fp8(M, N, K, fmts):
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    sa, sb = fp8.DelayedScale(fmts[0], "cuda"), fp8.DelayedScale(fmts[1], "cuda")
    sa.prepare(a, 0)
    sb.prepare(b, 0)
    a_op, _ = fp8.quantize(a, sa)
    b_op, _ = fp8.quantize(b, sb)
    for out_dtype in (torch.bfloat16, torch.float32):
        d = fp8.gemm(a_op, b_op, out_dtype=out_dtype)
        torch.cuda.synchronize()
        _lib.check_status("gemm_fp8")
        ref = fp8.dequantize(a_op) @ fp8.dequantize(b_op).t()
        tol = (2e-2 if out_dtype == torch.bfloat16 else 1e-3) * ref.abs().max().item()
        assert (d.float() - ref).abs().max().item() <= tol
        # per-tile relative error: a wrong tile far from the maximum must not pass
        e = (d.float() - ref).reshape(M // 128, 128, N // 128, 128).norm(dim=(1, 3))
        r = ref.reshape(M // 128, 128, N // 128, 128).norm(dim=(1, 3))
        assert (e / r).max().item() < (1e-2 if out_dtype == torch.bfloat16 else 1e-4)
    acc = torch.ones(M, N, device="cuda")
    fp8.gemm(a_op, b_op, out=acc, accumulate=True)
    torch.cuda.synchronize()
    assert (acc - (ref + 1)).abs().max().item() < 2e-3 * ref.abs().max().item()


def test_fp8_linear_training_triple_matches_cpu_emulation():
    torch.manual_seed(3)
    x = torch.randn(512, 256).bfloat16()
    w = (torch.randn(384, 256) * 0.05).bfloat16()
    dy = torch.randn(512, 384).bfloat16()
    res = {}
    for dev in ("cpu", "cuda"):
        xx, ww = x.detach().clone().to(dev).requires_grad_(True), w.detach().clone().to(dev).requires_grad_(True)
        y = F.linear(xx, ww, precision="fp8")
        y.backward(dy.to(dev))
        res[dev] = [t.detach().float().cpu() for t in (y, xx.grad, ww.grad)]
    torch.cuda.synchronize()
    _lib.check_status("fp8 linear")
    for a, b in zip(res["cuda"], res["cpu"]):
        assert (a - b).norm() / b.norm() < 1e-2
