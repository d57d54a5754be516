"""Jagged HSTU attention kernels (forward / backward) against the eager fp32 oracle."""
import pytest
import torch

from mlperf_training_b200.ops import _lib
from mlperf_training_b200.ops.hstu_ops import hstu_attention, hstu_attention_reference

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("lengths,targets,ctx", [
    ([128], None, 0),
    ([17, 300, 1, 513], None, 0),
    ([64, 257, 130], [1, 1, 1], 0),
    ([200, 40, 384], [1, 3, 2], 8),
])
@pytest.mark.parametrize("via_uvqk", [False, True])
def test_hstu_attention_fwd_bwd(lengths, targets, ctx, via_uvqk):
    torch.manual_seed(sum(lengths))
    H, D, N = 4, 128, 1024
    L = sum(lengths)
    offs = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    nt = None if targets is None else torch.tensor(targets, dtype=torch.int32)
    if via_uvqk:
        uvqk = torch.randn(L, 4 * H * D, device="cuda").bfloat16()
        v = uvqk[:, H * D:2 * H * D].unflatten(-1, (H, D))
        q = uvqk[:, 2 * H * D:3 * H * D].unflatten(-1, (H, D))
        k = uvqk[:, 3 * H * D:].unflatten(-1, (H, D))
    else:
        q, k, v = (torch.randn(L, H, D, device="cuda").bfloat16() for _ in range(3))
    alpha = D ** -0.5
    qg, kg, vg = (t.detach().clone().contiguous().requires_grad_(True) if not via_uvqk else t.detach().requires_grad_(True)
                  for t in (q, k, v))
    out = hstu_attention(qg, kg, vg, offs.cuda(), N, alpha, None if nt is None else nt.cuda(), ctx)
    do = torch.randn_like(out)
    out.backward(do)
    torch.cuda.synchronize()
    _lib.check_status("hstu attention")
    qf, kf, vf = (t.detach().float().cpu().requires_grad_(True) for t in (q, k, v))
    ref = hstu_attention_reference(qf, kf, vf, offs, N, alpha, nt, ctx)
    ref.backward(do.float().cpu())
    sc = ref.abs().max().item() + 1e-9
    assert (out.float().cpu() - ref.detach()).abs().max().item() < 3e-2 * sc + 1e-4
    for name, got, want in (("dq", qg.grad, qf.grad), ("dk", kg.grad, kf.grad), ("dv", vg.grad, vf.grad)):
        g = got.float().cpu()
        s = want.abs().max().item() + 1e-9
        assert (g - want).abs().max().item() < 4e-2 * s + 1e-5, name


@pytest.mark.parametrize("lengths,targets,ctx", [
    ([128], None, 0),
    ([17, 300, 1, 513], None, 0),
    ([200, 40, 384], [1, 3, 2], 8),
])
@pytest.mark.parametrize("via_uvqk", [False, True])
def test_hstu_attention_fp8_forward(lengths, targets, ctx, via_uvqk):
    """e4m3 forward against the eager emulation that rounds Q, K, V and the activation the same way, and against
    the fp32 oracle within quantisation error; the backward still runs (bf16 kernels)."""
    from mlperf_training_b200.ops.hstu_ops import hstu_attention_fp8_reference
    torch.manual_seed(sum(lengths) + 1)
    H, D, N = 4, 128, 1024
    L = sum(lengths)
    offs = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    nt = None if targets is None else torch.tensor(targets, dtype=torch.int32)
    if via_uvqk:
        uvqk = torch.randn(L, 4 * H * D, device="cuda").bfloat16()
        v = uvqk[:, H * D:2 * H * D].unflatten(-1, (H, D))
        q = uvqk[:, 2 * H * D:3 * H * D].unflatten(-1, (H, D))
        k = uvqk[:, 3 * H * D:].unflatten(-1, (H, D))
    else:
        q, k, v = (torch.randn(L, H, D, device="cuda").bfloat16() for _ in range(3))
    alpha = D ** -0.5
    qg, kg, vg = (t.detach().requires_grad_(True) for t in (q, k, v))
    out = hstu_attention(qg, kg, vg, offs.cuda(), N, alpha, None if nt is None else nt.cuda(), ctx, precision="fp8")
    out.backward(torch.randn_like(out))
    torch.cuda.synchronize()
    _lib.check_status("hstu attention fp8")
    assert qg.grad is not None and torch.isfinite(qg.grad.float()).all()
    emu = hstu_attention_fp8_reference(q.float().cpu(), k.float().cpu(), v.float().cpu(), offs, N, alpha, nt, ctx)
    ref = hstu_attention_reference(q.float().cpu(), k.float().cpu(), v.float().cpu(), offs, N, alpha, nt, ctx)
    got = out.float().cpu()
    sc = ref.abs().max().item() + 1e-9
    assert (got - emu).abs().max().item() < 2e-2 * sc + 1e-5          # a score on a rounding boundary may flip one code
    assert ((got - ref).norm() / ref.norm()).item() < 0.08


def test_rowwise_adagrad_and_segment_sum_kernels():
    from mlperf_training_b200.parallel.embedding import ShardedEmbedding
    torch.manual_seed(0)
    t = ShardedEmbedding(4096, 256, device="cuda", dtype=torch.bfloat16, lr=0.05, seed=3)
    w0 = t.weight.float().clone()
    ids = torch.randint(0, 4096, (3000,), device="cuda")
    out = t.lookup(ids)
    assert torch.equal(out, t.weight[ids])
    w = torch.randn(3000, 256, device="cuda").bfloat16().float()     # the gradient reaches the table in bf16
    (out.float() * w).sum().backward()
    torch.cuda.synchronize()
    u, inv = torch.unique(ids, return_inverse=True)
    g = torch.zeros(u.numel(), 256, device="cuda").index_add_(0, inv, w)
    st = (g * g).mean(-1)
    ref = w0.clone()
    ref[u] = (w0[u] - 0.05 * g / (st.sqrt()[:, None] + t.eps)).bfloat16().float()
    assert (t.weight.float() - ref).abs().max().item() < 1e-2
    assert torch.allclose(t.state[u], st, rtol=1e-4, atol=1e-6)
    # segment sum of sorted duplicate rows
    src = torch.randn(1000, 256, device="cuda").bfloat16()
    seg = torch.tensor([0, 1, 5, 5, 400, 1000], device="cuda")
    o = torch.empty(5, 256, device="cuda")
    _lib.call("b200_segment_sum_rows", _lib.ptr(src), _lib.ptr(seg), 5, 256, _lib.ptr(o), _lib.stream_ptr())
    want = torch.stack([src[a:b].float().sum(0) for a, b in zip(seg[:-1].tolist(), seg[1:].tolist())])
    assert torch.allclose(o, want, rtol=1e-4, atol=1e-3)


def test_hstu_train_steps_on_gpu():
    import io
    from mlperf_training_b200.trainer.hstu import run
    before = _lib.launch_count()
    exp = dict(batch_per_gpu=16, train_steps=30, dense_lr=2e-3, sparse_lr=0.05, eval_interval_steps=15, num_eval_batches=2,
               model=dict(layers=2, dim=256, heads=2, d_qk=128, d_v=128, max_seq_len=512, dtype="bf16", mlp_hidden=64,
                          num_positions=512, num_time_buckets=128),
               embedding=dict(rows=5000, dim=128), data=dict(length_median=100, length_min=8, length_max=400))
    out = run(exp, device="cuda", stream=io.StringIO())
    _lib.check_status("hstu run")
    assert _lib.launch_count() > before
    assert all(l == l for l in out["losses"])
    assert sum(out["losses"][-5:]) < sum(out["losses"][:5])
    assert out["aucs"][-1] > 0.55


def test_hstu_multi_table_train_steps_on_gpu():
    """The eleven-table feature set through the run loop on the GPU kernels: one sorted / deduplicated lookup per table,
    additional-feature branch, contextual tokens, row-wise Adagrad in backward."""
    import io
    from mlperf_training_b200.trainer.hstu import run
    exp = dict(batch_per_gpu=16, train_steps=24, dense_lr=2e-3, sparse_lr=0.05, eval_interval_steps=12, num_eval_batches=2,
               model=dict(layers=2, dim=256, heads=2, d_qk=128, d_v=128, max_seq_len=512, dtype="bf16", mlp_hidden=64,
                          num_positions=1024, num_time_buckets=128),
               embedding=dict(rows=5000, dim=128, tables="yambda", table_scale=2000),
               data=dict(length_median=100, length_min=8, length_max=400))
    out = run(exp, device="cuda", stream=io.StringIO())
    _lib.check_status("hstu multi-table run")
    assert all(l == l for l in out["losses"])
    assert sum(out["losses"][-5:]) < sum(out["losses"][:5])


@pytest.mark.parametrize("T,D,pitch", [(1000, 512, 2048), (37, 256, 256), (4099, 768, 1536)])
def test_gate_cat_kernel_against_fp32_reference(T, D, pitch):
    """silu(u) | attn | silu(u) * LN(attn): forward and all four gradients against fp32 autograd."""
    from mlperf_training_b200.ops.hstu_ops import GateCatFn, gate_cat_eligible
    torch.manual_seed(T)
    wide = torch.randn(T, pitch, device="cuda").bfloat16()
    u_raw = wide[:, :D]
    attn = (torch.randn(T, D, device="cuda") * 2 + 0.3).bfloat16()
    w = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16()
    b = (0.1 * torch.randn(D, device="cuda")).bfloat16()
    dcat = torch.randn(T, 3 * D, device="cuda").bfloat16()
    assert gate_cat_eligible(u_raw, attn)
    leaves = [t.clone().requires_grad_(True) for t in (u_raw.contiguous(), attn, w, b)]
    uk = wide.clone().requires_grad_(True)
    ak, wk, bk = (t.clone().requires_grad_(True) for t in (attn, w, b))
    cat = GateCatFn.apply(uk[:, :D], ak, wk, bk, 1e-6)
    cat.backward(dcat)
    torch.cuda.synchronize()
    _lib.check_status("gate_cat")
    uf, af, wf, bf = (t.detach().float().requires_grad_(True) for t in leaves)
    u = torch.nn.functional.silu(uf)
    n = torch.nn.functional.layer_norm(af, (D,), wf, bf, 1e-6)
    ref = torch.cat([u, af, u * n], dim=1)
    ref.backward(dcat.float())

    def close(got, want, tol, what):
        err = (got.float() - want).abs().max().item()
        scale = want.abs().max().item() + 1e-6
        assert err <= tol * scale, f"{what}: err {err} scale {scale}"
    close(cat, ref.detach(), 2e-2, "cat")
    close(uk.grad[:, :D], uf.grad, 2e-2, "du_raw")
    assert uk.grad[:, D:].abs().max().item() == 0 if pitch > D else True
    close(ak.grad, af.grad, 2e-2, "dattn")
    close(wk.grad, wf.grad, 2e-2, "dw")
    close(bk.grad, bf.grad, 2e-2, "db")


def test_stu_layer_fused_glue_matches_eager_glue():
    from mlperf_training_b200.models.hstu import HSTUConfig, STULayer
    cfg = HSTUConfig(layers=1, dim=512, heads=4, d_qk=128, d_v=128, max_seq_len=512, emb_dim=64, dtype="bf16", precision="bf16",
                     linear_dropout=0.0)
    torch.manual_seed(0)
    layer = STULayer(cfg, torch.bfloat16, "cuda")
    lengths = [100, 256, 28]
    rows = 384
    offs = torch.tensor([0, 100, 356, 384], dtype=torch.int32, device="cuda")
    nt = torch.tensor([1, 2, 1], dtype=torch.int32, device="cuda")
    x0 = torch.randn(rows, 512, device="cuda").bfloat16()
    dy = torch.randn(rows, 512, device="cuda").bfloat16()
    outs = []
    for fuse in (False, True):
        layer.fuse_glue = fuse
        layer.zero_grad(set_to_none=True)
        x = x0.clone().requires_grad_(True)
        y = layer(x, offs, nt, rows)
        y.backward(dy)
        outs.append((y.detach().float(), x.grad.float(), layer.out_norm_w.grad.float(), layer.uvqk_weight.grad.float()))
    torch.cuda.synchronize()
    _lib.check_status("stu_layer")
    for a, b, what in zip(outs[0], outs[1], ("y", "dx", "dnorm_w", "duvqk_w")):
        err = (a - b).abs().max().item()
        assert err <= 2e-2 * (a.abs().max().item() + 1e-6), f"{what}: {err}"


def test_gate_cat_dropout_mask_is_regenerated_in_backward():
    from mlperf_training_b200.ops.hstu_ops import GateCatFn
    torch.manual_seed(11)
    T, D, p = 3000, 512, 0.25
    wide = torch.randn(T, 2048, device="cuda").bfloat16()
    attn = (torch.randn(T, D, device="cuda") * 2 + 0.3).bfloat16()
    w = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16()
    b = (0.1 * torch.randn(D, device="cuda")).bfloat16()
    dcat = torch.randn(T, 3 * D, device="cuda").bfloat16()
    plain = GateCatFn.apply(wide[:, :D], attn, w, b, 1e-6, 0.0)
    uk = wide.clone().requires_grad_(True)
    ak, wk, bk = (t.clone().requires_grad_(True) for t in (attn, w, b))
    dropped = GateCatFn.apply(uk[:, :D], ak, wk, bk, 1e-6, p)
    dropped.backward(dcat)
    torch.cuda.synchronize()
    _lib.check_status("gate_cat_dropout")
    keep = (dropped != 0) | (plain == 0)
    frac = 1.0 - keep.float().mean().item()
    assert abs(frac - p) < 0.01, frac
    for sec in range(3):                                   # every section gets its own bits
        f = 1.0 - keep[:, sec * D:(sec + 1) * D].float().mean().item()
        assert abs(f - p) < 0.02, (sec, f)
    want = plain.float() / (1 - p) * keep
    assert (dropped.float() - want).abs().max().item() <= 2 ** -6 * want.abs().max().item()
    # another call draws another mask
    again = GateCatFn.apply(wide[:, :D], attn, w, b, 1e-6, p)
    assert ((again != 0) != (dropped != 0)).float().mean().item() > 0.2
    # backward against fp32 autograd through the same mask
    uf, af, wf, bf = (t.detach().float().requires_grad_(True) for t in (wide[:, :D].contiguous(), attn, w, b))
    u = torch.nn.functional.silu(uf)
    n = torch.nn.functional.layer_norm(af, (D,), wf, bf, 1e-6)
    (torch.cat([u, af, u * n], dim=1) * keep / (1 - p)).backward(dcat.float())
    for got, ref, what in ((uk.grad[:, :D], uf.grad, "du_raw"), (ak.grad, af.grad, "dattn"), (wk.grad, wf.grad, "dw"),
                           (bk.grad, bf.grad, "db")):
        err = (got.float() - ref).abs().max().item()
        assert err <= 2e-2 * (ref.abs().max().item() + 1e-6), f"{what}: {err}"


def test_expand_rows_backward_is_a_segment_sum():
    """``src[seq]`` over ascending groups: gather forward, per-group sum backward, against index arithmetic."""
    from mlperf_training_b200.ops import functional as F
    torch.manual_seed(3)
    lens = torch.tensor([5, 0, 300, 1, 77, 2000])
    offs = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)]).to(torch.int32).cuda()
    seq = torch.repeat_interleave(torch.arange(lens.numel()), lens).cuda()
    src = torch.randn(lens.numel(), 512, device="cuda").bfloat16().requires_grad_(True)
    out = F.expand_rows(src, seq, offs)
    assert torch.equal(out, src.detach()[seq])
    g = torch.randn_like(out)
    out.backward(g)
    torch.cuda.synchronize()
    _lib.check_status("expand rows")
    want = torch.zeros(lens.numel(), 512, device="cuda").index_add_(0, seq, g.float())
    assert (src.grad.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item()
    assert src.grad[1].abs().max() == 0


def test_hstu_interleaved_preprocessor_and_generated_mlps_on_gpu():
    """Content and action tokens interleaved (sequences twice as long), content / action MLPs generated from the
    contextual features: the eleven-table run trains on the GPU kernels."""
    import io
    from mlperf_training_b200.trainer.hstu import run
    exp = dict(batch_per_gpu=8, train_steps=16, dense_lr=2e-3, sparse_lr=0.05, eval_interval_steps=8, num_eval_batches=2,
               model=dict(layers=2, dim=256, heads=2, d_qk=128, d_v=128, max_seq_len=512, dtype="bf16", mlp_hidden=64,
                          num_positions=2048, num_time_buckets=128, preprocessor="interleave",
                          contextualized_mlp="parameterized"),
               embedding=dict(rows=5000, dim=128, tables="yambda", table_scale=2000),
               data=dict(length_median=100, length_min=8, length_max=400))
    out = run(exp, device="cuda", stream=io.StringIO())
    _lib.check_status("hstu interleaved run")
    # (eight candidates per step: the per-step loss is too noisy to compare ends; the CPU run of this configuration
    # moves in the same band)
    assert len(out["losses"]) == 16 and all(l == l and 0.0 < l < 1.5 for l in out["losses"])


def test_column_wise_table_single_rank_on_gpu():
    from mlperf_training_b200.parallel.embedding import ColumnShardedEmbedding
    t = ColumnShardedEmbedding(300, 64, device="cuda", dtype=torch.bfloat16, lr=0.1, seed=2)
    ids = torch.tensor([3, 3, 7, 299, 0], device="cuda")
    w0 = t.weight.clone()
    rows = t.lookup(ids)
    assert torch.equal(rows, w0[ids])
    rows.float().sum().backward()
    torch.cuda.synchronize()
    _lib.check_status("column-wise table")
    # row 3 saw a gradient of 2 per column, the others of 1: Adagrad's first step moves each by lr (sum = mean g^2)
    moved = (w0.float() - t.weight.float())
    assert torch.allclose(moved[[3, 7, 299, 0]], torch.full((4, 64), 0.1, device="cuda"), atol=2e-3)
    assert float(moved[[1, 2, 100]].abs().max()) == 0
