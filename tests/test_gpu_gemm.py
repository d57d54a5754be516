"""tcgen05 bf16 GEMM against a plain fp32 PyTorch matmul of the same bf16 operands."""
import pytest
import torch

from mlperf_training_b200.ops import _lib, kernels

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    am = a.float().t() if a_mn else a.float()
    bm = b.float() if b_mn else b.float().t()
    return am @ bm


def _check(d, ref, K, what):
    err = (d.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    tol = 2e-2 * scale if d.dtype == torch.bfloat16 else 2e-3 * scale
    _lib.check_status(what)
    assert err <= tol, f"{what}: max err {err} vs tol {tol} (scale {scale})"


SHAPES = [(128, 256, 64), (256, 256, 128), (128, 128, 256), (384, 512, 192), (300, 520, 136), (1024, 1024, 1024),
          (2048, 4096, 512), (136, 72, 64)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    torch.manual_seed(M * 7 + N * 3 + K)
    dev = "cuda"
    a = torch.randn((K, M) if a_mn else (M, K), device=dev).bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device=dev).bfloat16()
    d = kernels.gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn)
    torch.cuda.synchronize()
    _check(d, _ref(a, b, a_mn, b_mn), K, f"gemm {M}x{N}x{K} a_mn={a_mn} b_mn={b_mn}")


def test_gemm_fp32_out_and_accumulate():
    torch.manual_seed(1)
    M, N, K = 512, 768, 320
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    ref = _ref(a, b, False, False)
    d = kernels.gemm(a, b, out_dtype=torch.float32)
    torch.cuda.synchronize()
    _check(d, ref, K, "fp32 out")
    acc = torch.full((M, N), 0.5, device="cuda", dtype=torch.float32)
    kernels.gemm(a, b, out=acc, accumulate=True)
    kernels.gemm(a, b, out=acc, accumulate=True)
    torch.cuda.synchronize()
    _check(acc, 2 * ref + 0.5, K, "fp32 accumulate x2")
    accb = torch.zeros((M, N), device="cuda", dtype=torch.bfloat16)
    kernels.gemm(a, b, out=accb, accumulate=True)
    torch.cuda.synchronize()
    _check(accb, ref, K, "bf16 accumulate")


def test_gemm_bias_residual_alpha():
    torch.manual_seed(2)
    M, N, K = 300, 264, 128
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16()
    d = kernels.gemm(a, b, bias=bias, residual=res, alpha=0.5)
    torch.cuda.synchronize()
    ref = 0.5 * _ref(a, b, False, False) + bias.float() + res.float()
    _check(d, ref, K, "bias+residual+alpha")


def test_gemm_strided_views():
    torch.manual_seed(3)
    M, N, K = 256, 384, 128
    big_a = torch.randn(M, K + 64, device="cuda").bfloat16()
    a = big_a[:, 32:32 + K]  # pitch K+64, base offset 64 bytes
    b = torch.randn(N, K, device="cuda").bfloat16()
    out_big = torch.zeros(M, N + 128, device="cuda", dtype=torch.bfloat16)
    out = out_big[:, 64:64 + N]
    kernels.gemm(a, b, out=out)
    torch.cuda.synchronize()
    _check(out, _ref(a, b, False, False), K, "strided")
    assert out_big[:, :64].abs().max().item() == 0 and out_big[:, 64 + N:].abs().max().item() == 0


def test_gemm_deterministic():
    torch.manual_seed(4)
    a = torch.randn(1024, 512, device="cuda").bfloat16()
    b = torch.randn(768, 512, device="cuda").bfloat16()
    d1 = kernels.gemm(a, b)
    d2 = kernels.gemm(a, b)
    torch.cuda.synchronize()
    assert torch.equal(d1, d2)
