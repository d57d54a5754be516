"""CPU bodies of the raw operators against autograd / torch built-ins (they are the oracles of
the GPU tests, so they are checked independently here)."""
import math

import pytest

import torch
import torch.nn.functional as F

from mlperf_training_b200.ops import kernels


def test_gemm_cpu_layouts():
    torch.manual_seed(0)
    x, w, dy = torch.randn(6, 8).bfloat16(), torch.randn(5, 8).bfloat16(), torch.randn(6, 5).bfloat16()
    assert torch.allclose(kernels.gemm(x, w).float(), x.float() @ w.float().t(), atol=5e-2)
    assert torch.allclose(kernels.gemm(dy, w, b_mn_major=True).float(), dy.float() @ w.float(), atol=5e-2)
    assert torch.allclose(kernels.gemm(dy, x, a_mn_major=True, b_mn_major=True).float(),
                          dy.float().t() @ x.float(), atol=5e-2)


def test_norm_bwd_matches_autograd():
    torch.manual_seed(1)
    T, D = 7, 32
    for layer_norm, swish in ((False, False), (True, False), (True, True)):
        x = torch.randn(T, D)
        w = torch.randn(D)
        b = torch.randn(D) if layer_norm else None
        dy = torch.randn(T, D)
        y, h, mean, rstd = kernels.norm_fwd(x, w, b, 1e-5, layer_norm=layer_norm, swish=swish)
        dx, dw, db = kernels.norm_bwd(dy, h, w, b, mean, rstd, layer_norm=layer_norm, swish=swish)
        xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        br = None if b is None else b.clone().requires_grad_(True)
        if layer_norm:
            n = F.layer_norm(xr, (D,), wr, br, 1e-5)
        else:
            n = xr * torch.rsqrt((xr * xr).mean(-1, keepdim=True) + 1e-5) * wr
        yr = xr * torch.sigmoid(n) if swish else n
        assert torch.allclose(y, yr, atol=1e-5)
        yr.backward(dy)
        assert torch.allclose(dx, xr.grad, atol=1e-4)
        assert torch.allclose(dw, wr.grad, atol=1e-4)
        if layer_norm:
            assert torch.allclose(db, br.grad, atol=1e-4)


def test_rope_is_rotation():
    T, S, H, D = 10, 5, 2, 16
    x = torch.randn(T, H * D)
    cos, sin = kernels.rope_tables(S, D, 10000.0, "cpu")
    y = kernels.rope_(x.clone(), cos, sin, col0=0, n_heads=H, head_dim=D, seq_len=S)
    assert torch.allclose(y.view(T, H, D).norm(dim=-1), x.view(T, H, D).norm(dim=-1), atol=1e-5)
    back = kernels.rope_(y.clone(), cos, sin, col0=0, n_heads=H, head_dim=D, seq_len=S, backward=True)
    assert torch.allclose(back, x, atol=1e-5)


def test_swiglu_bwd_matches_autograd():
    gu = torch.randn(4, 12, requires_grad=True)
    a = F.silu(gu[:, :6]) * gu[:, 6:]
    da = torch.randn(4, 6)
    a.backward(da)
    assert torch.allclose(kernels.swiglu_bwd(da, gu.detach()), gu.grad, atol=1e-5)


def test_cross_entropy_matches_torch():
    T, V = 9, 40
    logits = torch.randn(T, V)
    labels = torch.randint(0, V, (T,))
    labels[2] = -100
    ref_in = logits.clone().requires_grad_(True)
    ref = F.cross_entropy(ref_in, labels, reduction="sum", ignore_index=-100)
    ref.backward()
    work = logits.clone()
    loss = kernels.cross_entropy_(work, labels, 1.0)
    assert torch.allclose(loss.sum(), ref, atol=1e-4)
    assert torch.allclose(work, ref_in.grad, atol=1e-5)


def test_adamw_matches_torch():
    torch.manual_seed(2)
    p = torch.randn(50)
    ref = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros(50), torch.zeros(50)
    mine = p.clone()
    for step in (1, 2, 3):
        g = torch.randn(50)
        ref.grad = g.clone()
        opt.step()
        kernels.adamw_(mine, g, m, v, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
    assert torch.allclose(mine, ref.data, atol=1e-5)


def test_attention_reference_matches_sdpa_and_sink():
    torch.manual_seed(3)
    B, S, Hq, Hkv, D = 2, 16, 4, 2, 8
    q, k, v = torch.randn(B, S, Hq, D), torch.randn(B, S, Hkv, D), torch.randn(B, S, Hkv, D)
    o, lse = kernels.attention_reference(q, k, v, scale=1 / math.sqrt(D), causal=True)
    ref = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2).repeat_interleave(2, 1),
                                         v.transpose(1, 2).repeat_interleave(2, 1), is_causal=True).transpose(1, 2)
    assert torch.allclose(o, ref, atol=1e-5)
    # a very negative sink changes nothing; a large one shrinks the output
    o2, _ = kernels.attention_reference(q, k, v, scale=1 / math.sqrt(D), causal=True, sink=torch.full((Hq,), -1e4))
    assert torch.allclose(o2, o, atol=1e-5)
    o3, _ = kernels.attention_reference(q, k, v, scale=1 / math.sqrt(D), causal=True, sink=torch.full((Hq,), 20.0))
    assert o3.abs().max() < 1e-3 * max(o.abs().max(), 1.0) + 1e-3
    # window: each query sees at most `window` keys
    ow, _ = kernels.attention_reference(q, k, v, scale=1.0, causal=True, window=1)
    assert torch.allclose(ow, v.repeat_interleave(2, 2), atol=1e-5)


def test_mxfp8_emulation_roundtrip():
    from mlperf_training_b200.ops import mxfp8
    torch.manual_seed(5)
    x = (torch.randn(128, 256) * 3).bfloat16()
    row, col = mxfp8.quantize(x, row_tile=128, col_tile=224)
    assert row.q.shape == (128, 256) and col.q.shape == (256, 128)
    d = mxfp8.dequantize(row)
    assert (d - x.float()).abs().max() <= x.float().abs().max() * 0.07
    assert torch.allclose(mxfp8.dequantize(col), mxfp8.dequantize(mxfp8.quantize(x.t().contiguous(), row_tile=224)[0]))
    # scales are the smallest powers of two that keep the block inside +-448
    s = torch.exp2(row.sf.float() - 127)
    amax = x.float().abs().view(128, 8, 32).amax(-1)
    assert (amax / s <= 448).all() and ((amax / s > 224) | (amax == 0)).all()
    y = mxfp8.gemm(row, row, out_dtype=torch.float32)
    assert torch.allclose(y, d @ d.t(), atol=1e-3)
    # the flat atom layout addresses every scale exactly once
    idx = mxfp8.sf_index(448, 256, 224, "cpu")
    assert idx.unique().numel() == idx.numel() and int(idx.max()) < mxfp8.sf_bytes(448, 256, 224)


def test_hstu_mask_rules():
    from mlperf_training_b200.ops.hstu_ops import valid_mask
    m = valid_mask(5).int()
    assert torch.equal(m, torch.tril(torch.ones(5, 5)).int())                 # plain causal
    m = valid_mask(6, n_targets=2)                                            # rows 4, 5 are targets
    assert m[4, :4].all() and m[5, :4].all() and m[4, 4] and m[5, 5] and not m[5, 4] and not m[4, 5]
    m = valid_mask(7, n_targets=1, contextual=3)                              # rows 0..2 contextual
    assert m[0, :6].all() and not m[0, 6]                                     # contextual rows see all history
    assert m[3, :3].all() and m[3, 3] and not m[3, 4]
    assert m[6, :6].all() and m[6, 6]


def test_activation_recompute_matches_plain_backward():
    import torch
    from mlperf_training_b200.models.gpt import GPT, GPTConfig
    kw = dict(n_layers=3, hidden=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn_hidden=128, vocab_size=256, seq_len=32,
              dtype="fp32")
    tok = torch.randint(0, 256, (2, 33), generator=torch.Generator().manual_seed(0))
    out = []
    for rc, n in (("none", 0), ("full", 2), ("full", 0)):
        m = GPT(GPTConfig(recompute=rc, recompute_layers=n, **kw), seed=1)
        loss = m(tok[:, :-1], tok[:, 1:])
        loss.backward()
        out.append((loss.item(), [p.grad.clone() for p in m.parameters()]))
    for l, g in out[1:]:
        assert l == out[0][0]
        assert all(torch.equal(a, b) for a, b in zip(g, out[0][1]))


def test_adamw_bf16_moments_track_fp32_moments():
    torch.manual_seed(5)
    n = 4096
    p32, p16 = torch.randn(n), None
    p16 = p32.clone()
    m32, v32 = torch.zeros(n), torch.zeros(n)
    m16, v16 = torch.zeros(n, dtype=torch.bfloat16), torch.zeros(n, dtype=torch.bfloat16)
    for step in range(1, 9):
        g = torch.randn(n)
        kw = dict(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
        kernels.adamw_(p32, g, m32, v32, **kw)
        kernels.adamw_(p16, g, m16, v16, **kw)
    assert m16.dtype == torch.bfloat16 and v16.dtype == torch.bfloat16
    # one bf16 rounding per step on each moment: relative error of a few 2^-8, the weights stay close
    assert (m16.float() - m32).abs().max().item() < 0.03
    assert ((v16.float() - v32).abs() / v32).max().item() < 0.03
    assert (p16 - p32).abs().max().item() < 5e-3
    with pytest.raises(ValueError):
        kernels.adamw_(p16, g, m16, v32, **kw)


def test_engine_bf16_moments_train():
    from mlperf_training_b200.models.gpt import GPT, GPTConfig
    from mlperf_training_b200.parallel.engine import OptimConfig, ZeroEngine
    cfg = GPTConfig(n_layers=2, hidden=32, n_heads=2, n_kv_heads=1, head_dim=16, ffn_hidden=64, vocab_size=64, seq_len=16, dtype="fp32")
    tok = torch.randint(0, 64, (4, 17), generator=torch.Generator().manual_seed(0))
    curves = []
    for md in (torch.float32, torch.bfloat16):
        model = GPT(cfg, seed=3)
        eng = ZeroEngine(model, OptimConfig(lr=3e-3, weight_decay=0.0, clip_grad=1.0, moment_dtype=md))
        assert all(b.m.dtype == md and b.v.dtype == md for b in eng.buckets)
        losses = []
        for _ in range(12):
            loss = model(tok[:, :-1], tok[:, 1:])
            loss.backward()
            eng.step()
            losses.append(loss.item())
        curves.append(losses)
        eng.load_optimizer_state(eng.optimizer_state())
    assert curves[1][-1] < curves[1][0] - 0.3
    assert abs(curves[1][-1] - curves[0][-1]) < 0.05


def test_run_config_selects_moment_dtype():
    from mlperf_training_b200.trainer.loop import RunConfig, _moment_dtype
    assert _moment_dtype(RunConfig()) == torch.float32
    assert _moment_dtype(RunConfig(use_precision_aware_optimizer=True, exp_avg_dtype="bf16", exp_avg_sq_dtype="bf16")) == torch.bfloat16
    assert _moment_dtype(RunConfig(use_precision_aware_optimizer=False, exp_avg_dtype="bf16", exp_avg_sq_dtype="bf16")) == torch.float32
    with pytest.raises(ValueError):
        _moment_dtype(RunConfig(use_precision_aware_optimizer=True, exp_avg_dtype="fp16", exp_avg_sq_dtype="bf16"))


def test_grouped_mlp_block_scaled_emulation_close_to_bf16():
    """The block-scaled expert MLP (eager emulation: e4m3 codes, one power-of-two scale per 32) stays within
    quantisation error of the bf16 grouped path, forward and all three gradients, with an empty expert."""
    from mlperf_training_b200.ops import moe_ops as M
    torch.manual_seed(0)
    T, k, E, D, F = 96, 2, 4, 192, 192
    x = torch.randn(T, D).bfloat16()
    logits = torch.randn(T, E)
    logits[:, 2] -= 100.0
    w1 = (torch.randn(E, 2 * F, D) * 0.05).bfloat16().requires_grad_()
    w2 = (torch.randn(E, D, F) * 0.05).bfloat16().requires_grad_()
    idx, w, counts = M.router_topk(logits, k)
    assert M.expert_precision("mxfp8", w1, w2) == "mxfp8"

    def run(prec):
        xx = x.clone().requires_grad_()
        w1.grad = w2.grad = None
        y = M.moe_experts(xx, idx, w, counts, w1, w2, prec)
        y.float().square().sum().backward()
        return y.detach().float(), xx.grad.float(), w1.grad.float().clone(), w2.grad.float().clone()

    ref = run("bf16")
    for u, v in zip(ref, run("mxfp8")):
        assert ((u - v).norm() / u.norm()).item() < 0.12
    assert w1.grad[2].abs().max() == 0
    # the narrower micro-scaled recipes run the same grouped path on operands rounded to their element grids
    assert M.expert_precision("mxfp4", w1, w2) == "mxfp4" and M.pad_rows("a6w4") == M.PAD_MX
    e8 = [((u - v).norm() / u.norm()).item() for u, v in zip(ref, run("mxfp8"))]
    e6 = [((u - v).norm() / u.norm()).item() for u, v in zip(ref, run("mxfp6"))]
    e4 = [((u - v).norm() / u.norm()).item() for u, v in zip(ref, run("mxfp4"))]
    assert all(a < b * 1.3 for a, b in zip(e8, e6)) and all(a < b for a, b in zip(e6, e4)) and max(e4) < 0.6
    assert w1.grad[2].abs().max() == 0 and w1._mx_stack[0][2] == "e2m1"
