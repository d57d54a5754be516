"""Bandwidth-bound kernels against their eager fp32 definitions (the CPU bodies in ops.kernels)."""
import pytest
import torch

from mlperf_training_b200.ops import _lib, kernels

pytestmark = pytest.mark.gpu


def _close(a, b, tol, what):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs().max().item()
    scale = b.abs().max().item() + 1e-6
    assert err <= tol * scale, f"{what}: err {err} scale {scale}"


@pytest.mark.parametrize("layer_norm,swish", [(False, False), (True, False), (True, True)])
@pytest.mark.parametrize("T,D", [(37, 512), (300, 4096), (64, 2880), (16, 256)])
def test_norm_fwd_bwd(layer_norm, swish, T, D):
    torch.manual_seed(T + D)
    x = torch.randn(T, D).bfloat16()
    res = torch.randn(T, D).bfloat16()
    w = (1 + 0.1 * torch.randn(D)).bfloat16()
    b = (0.1 * torch.randn(D)).bfloat16() if layer_norm else None
    dy = torch.randn(T, D).bfloat16()
    dres = torch.randn(T, D).bfloat16()
    y_c, h_c, mean_c, rstd_c = kernels.norm_fwd(x, w, b, 1e-5, layer_norm=layer_norm, swish=swish, residual=res)
    dx_c, dw_c, db_c = kernels.norm_bwd(dy, h_c, w, b, mean_c, rstd_c, layer_norm=layer_norm, swish=swish, dres=dres)
    g = lambda t: None if t is None else t.cuda()
    y_g, h_g, mean_g, rstd_g = kernels.norm_fwd(g(x), g(w), g(b), 1e-5, layer_norm=layer_norm, swish=swish,
                                                residual=g(res))
    dx_g, dw_g, db_g = kernels.norm_bwd(g(dy), h_g, g(w), g(b), mean_g, rstd_g, layer_norm=layer_norm, swish=swish,
                                        dres=g(dres))
    torch.cuda.synchronize()
    _close(h_g, h_c, 1e-6, "h")
    _close(y_g, y_c, 2e-2, "y")
    _close(rstd_g, rstd_c, 1e-4, "rstd")
    _close(dx_g, dx_c, 2e-2, "dx")
    _close(dw_g, dw_c, 2e-2, "dw")
    if layer_norm:
        _close(db_g, db_c, 2e-2, "db")
    # accumulate into existing fp32 grads
    dw_acc = torch.ones(D, device="cuda")
    kernels.norm_bwd(g(dy), h_g, g(w), g(b), mean_g, rstd_g, layer_norm=layer_norm, swish=swish, dw_out=dw_acc,
                     accumulate=True)
    _close(dw_acc - 1, kernels.norm_bwd(dy, h_c, w, b, mean_c, rstd_c, layer_norm=layer_norm, swish=swish)[1], 2e-2,
           "dw accumulate")


def test_rope_roundtrip_and_reference():
    torch.manual_seed(0)
    T, S, Hq, Hkv, D = 96, 48, 4, 2, 128
    row = (Hq + 2 * Hkv) * D
    qkv = torch.randn(T, row).bfloat16()
    cos, sin = kernels.rope_tables(S, D, 500000.0, "cpu")
    ref = qkv.clone()
    kernels.rope_(ref, cos, sin, col0=0, n_heads=Hq + Hkv, head_dim=D, seq_len=S)
    dev = qkv.cuda()
    kernels.rope_(dev, cos.cuda(), sin.cuda(), col0=0, n_heads=Hq + Hkv, head_dim=D, seq_len=S)
    _close(dev, ref, 1e-2, "rope fwd")
    kernels.rope_(dev, cos.cuda(), sin.cuda(), col0=0, n_heads=Hq + Hkv, head_dim=D, seq_len=S, backward=True)
    _close(dev, qkv, 2e-2, "rope roundtrip")
    assert torch.equal(dev[:, (Hq + Hkv) * D:].cpu(), qkv[:, (Hq + Hkv) * D:])


def test_swiglu_gelu():
    torch.manual_seed(1)
    T, F = 50, 1024
    gu = torch.randn(T, 2 * F).bfloat16()
    da = torch.randn(T, F).bfloat16()
    _close(kernels.swiglu_fwd(gu.cuda()), kernels.swiglu_fwd(gu), 1e-2, "swiglu fwd")
    _close(kernels.swiglu_bwd(da.cuda(), gu.cuda()), kernels.swiglu_bwd(da, gu), 2e-2, "swiglu bwd")
    x = torch.randn(T, F).bfloat16()
    _close(kernels.gelu_fwd(x.cuda()), kernels.gelu_fwd(x), 1e-2, "gelu fwd")
    _close(kernels.gelu_bwd(da.cuda(), x.cuda()), kernels.gelu_bwd(da, x), 2e-2, "gelu bwd")


def test_gather_scatter():
    torch.manual_seed(2)
    R, D, T = 1000, 256, 333
    table = torch.randn(R, D).bfloat16()
    ids = torch.randint(0, R, (T,))
    ids[5] = -1
    _close(kernels.gather_rows(table.cuda(), ids.cuda()), kernels.gather_rows(table, ids), 0, "gather")
    dy = torch.randn(T, D).bfloat16()
    g_c = kernels.scatter_add_rows(torch.zeros(R, D), ids, dy)
    g_g = kernels.scatter_add_rows(torch.zeros(R, D, device="cuda"), ids.cuda(), dy.cuda())
    _close(g_g, g_c, 1e-5, "scatter add")


@pytest.mark.parametrize("V", [2048, 32000, 128256])
def test_cross_entropy(V):
    torch.manual_seed(3)
    T = 24
    logits = (torch.randn(T, V) * 3).bfloat16()
    labels = torch.randint(0, V, (T,))
    labels[3] = -100
    lc = logits.clone()
    loss_c = kernels.cross_entropy_(lc, labels, 0.25)
    lg = logits.cuda()
    loss_g = kernels.cross_entropy_(lg, labels.cuda(), 0.25)
    torch.cuda.synchronize()
    _close(loss_g, loss_c, 2e-3, "loss")
    assert (lg.float().cpu() - lc.float()).abs().max().item() < 2e-3
    assert lg[3].abs().max().item() == 0


@pytest.mark.parametrize("n", [100003, 262144])
@pytest.mark.parametrize("p_bf16,g_bf16,use_master", [(True, False, False), (True, True, True), (False, False, False)])
def test_adamw_bf16_moments(p_bf16, g_bf16, use_master, n):
    """bf16 moments: the kernel against the fp32 PyTorch body applied to the same bf16 state (scalar tail
    and 4-wide paths); each stored moment may differ by one bf16 rounding."""
    torch.manual_seed(6)
    p = torch.randn(n)
    g = torch.randn(n) * 0.5
    pd = p.bfloat16() if p_bf16 else p.clone()
    gd = g.bfloat16() if g_bf16 else g.clone()
    state_c = dict(p=pd.clone(), g=gd.clone(), m=torch.zeros(n, dtype=torch.bfloat16), v=torch.zeros(n, dtype=torch.bfloat16),
                   master=pd.float().clone() if use_master else None)
    state_g = {k: (None if t is None else t.cuda()) for k, t in state_c.items()}
    for step in (1, 2, 3):
        for st in (state_c, state_g):
            kernels.adamw_(st["p"], st["g"], st["m"], st["v"], lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8,
                           weight_decay=0.1, step=step, master=st["master"])
    torch.cuda.synchronize()
    assert state_g["m"].dtype == torch.bfloat16
    _close(state_g["m"].float(), state_c["m"].float(), 2 ** -7, "m")
    _close(state_g["v"].float(), state_c["v"].float(), 2 ** -7, "v")
    _close(state_g["p"], state_c["p"], 1e-2 if p_bf16 else 1e-3, "p")
    _lib.check_status("elementwise")


@pytest.mark.parametrize("p_bf16,g_bf16,use_master", [(True, False, False), (True, True, True), (False, False, False)])
def test_adamw_and_clip(p_bf16, g_bf16, use_master):
    torch.manual_seed(4)
    n = 100003
    p = torch.randn(n)
    g = torch.randn(n) * 3
    pd = p.bfloat16() if p_bf16 else p.clone()
    gd = g.bfloat16() if g_bf16 else g.clone()
    state_c = dict(p=pd.clone(), g=gd.clone(), m=torch.zeros(n), v=torch.zeros(n),
                   master=pd.float().clone() if use_master else None)
    state_g = {k: (None if t is None else t.cuda()) for k, t in state_c.items()}
    ss_c, ss_g = torch.zeros(1), torch.zeros(1, device="cuda")
    for step in (1, 2, 3):
        for st, ss in ((state_c, ss_c), (state_g, ss_g)):
            kernels.sumsq(st["g"], ss)
            kernels.adamw_(st["p"], st["g"], st["m"], st["v"], lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8,
                           weight_decay=0.1, step=step, master=st["master"], sumsq_buf=ss, max_norm=1.0)
    torch.cuda.synchronize()
    _close(ss_g, ss_c, 1e-4, "sumsq")
    _close(state_g["m"], state_c["m"], 1e-4, "m")
    _close(state_g["v"], state_c["v"], 1e-4, "v")
    _close(state_g["p"], state_c["p"], 1e-2 if p_bf16 else 1e-5, "p")
    _lib.check_status("elementwise")


@pytest.mark.parametrize("B,S,D", [(2, 128, 256), (3, 256, 3072), (1, 64, 4096)])
def test_mmdit_glue_kernels_match_eager(B, S, D):
    """AdaLN modulation and gated residual (forward and backward) against the same functions on CPU."""
    from mlperf_training_b200.ops import functional as F
    torch.manual_seed(B * S + D)
    T = B * S
    x = torch.randn(T, D).bfloat16()
    mod = (torch.randn(B, 3 * D) * 0.5).bfloat16()
    y_in = torch.randn(T, D).bfloat16()
    dy = torch.randn(T, D).bfloat16()
    outs = {}
    for dev in ("cpu", "cuda"):
        xx = x.to(dev).clone().requires_grad_(True)
        mm = mod.to(dev).clone().requires_grad_(True)
        yy = y_in.to(dev).clone().requires_grad_(True)
        shift, scale, gate = mm.chunk(3, dim=-1)
        h = F.ln_modulate(xx, shift, scale, B, 1e-6)
        out = F.gate_residual(h, yy, gate, B)
        out.backward(dy.to(dev))
        outs[dev] = [t.detach().float().cpu() for t in (h, out, xx.grad, mm.grad, yy.grad)]
    torch.cuda.synchronize()
    _lib.check_status("mmdit glue")
    for name, a, b in zip(("h", "out", "dx", "dmod", "dy"), outs["cuda"], outs["cpu"]):
        err = (a - b).norm() / (b.norm() + 1e-12)
        assert err < 1e-2, (name, float(err))


def test_rope_bshd_matches_eager_rotation():
    from mlperf_training_b200.ops import functional as F
    from mlperf_training_b200.models.mmdit import rope_tables_nd
    torch.manual_seed(0)
    B, S, H, D = 2, 96, 4, 128
    ids = torch.stack([torch.zeros(S), torch.arange(S) // 8, torch.arange(S) % 8], -1)
    cos, sin = rope_tables_nd(ids, (16, 56, 56), 10000.0)
    x = torch.randn(B, S, H, D).bfloat16()
    g = torch.randn(B, S, H, D).bfloat16()
    res = {}
    for dev in ("cpu", "cuda"):
        xx = x.to(dev).clone().requires_grad_(True)
        y = F.rope_bshd(xx, cos.to(dev), sin.to(dev))
        y.backward(g.to(dev))
        res[dev] = (y.detach().float().cpu(), xx.grad.float().cpu())
    half = D // 2
    x1, x2 = x[..., :half].float(), x[..., half:].float()
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    want = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
    assert (res["cpu"][0] - want).abs().max() < 2e-2 and (res["cuda"][0] - want).abs().max() < 2e-2
    assert (res["cuda"][1] - res["cpu"][1]).abs().max() < 2e-2
