"""HSTU model pieces on CPU (fp32): targets-only last layer, contextual tokens, additional features,
multitask head."""
import torch

from mlperf_training_b200.data.hstu_synth import HSTUSyntheticData
from mlperf_training_b200.models.hstu import HSTU, MultitaskHead, tiny_hstu


def _batch(B=5, rows=200, seed=0):
    d = HSTUSyntheticData(rows, B, length_median=10, length_min=3, length_max=40, seed=seed)
    return d.batch_at(0)


def test_targets_only_last_layer_equals_full_layer_then_split():
    b = _batch()
    outs = []
    for tol in (False, True):
        cfg = tiny_hstu(targets_only_last=tol, input_dropout=0.0, linear_dropout=0.0)
        m = HSTU(cfg, "cpu", seed=3)
        g = torch.Generator().manual_seed(1)
        emb = torch.randn(b["rows"], cfg.emb_dim, generator=g)
        emb[b["total"]:] = 0
        emb.requires_grad_(True)
        loss, preds, labels = m(b, emb)
        loss.backward()
        outs.append((loss.detach(), preds, emb.grad.clone(), m.layers[-1].uvqk_weight.grad.clone()))
    for a, c in zip(outs[0], outs[1]):
        assert torch.allclose(a, c, atol=2e-5, rtol=1e-4), (a - c).abs().max()
    # with several targets per sample the layer falls back to the full form
    b2 = dict(b, max_targets=2)
    m = HSTU(tiny_hstu(targets_only_last=True, input_dropout=0.0, linear_dropout=0.0), "cpu", seed=3)
    assert torch.isfinite(m(b2, emb.detach())[0])


def test_contextual_tokens_and_additional_features():
    b = _batch(B=4)
    cfg = tiny_hstu(contextual=3, extra_features=2, input_dropout=0.0, linear_dropout=0.0)
    m = HSTU(cfg, "cpu", seed=2)
    g = torch.Generator().manual_seed(5)
    emb = torch.randn(b["rows"], cfg.emb_dim, generator=g)
    extra = torch.randn(b["rows"], 2 * cfg.emb_dim, generator=g)
    ctx = torch.randn(4, 3, cfg.emb_dim, generator=g).requires_grad_(True)
    loss, preds, labels = m(b, emb, extra_emb=extra, contextual_emb=ctx)
    loss.backward()
    assert torch.isfinite(loss) and preds.shape == labels.shape == (4,)
    assert ctx.grad.abs().sum() > 0 and m.ctx_weight.grad.abs().sum() > 0 and m.extra_mlp.l1.weight.grad.abs().sum() > 0
    # a contextual feature changes the prediction of its own sample only
    ctx2 = ctx.detach().clone()
    ctx2[1] += 1.0
    p2 = m(b, emb, extra_emb=extra, contextual_emb=ctx2)[1]
    changed = (p2 - preds).abs() > 1e-7
    assert changed.tolist() == [False, True, False, False]
    # the targets-only form sees the contextual rows like the full form does
    m_full = HSTU(tiny_hstu(contextual=3, extra_features=2, input_dropout=0.0, linear_dropout=0.0, targets_only_last=False), "cpu", seed=2)
    l_full = m_full(b, emb, extra_emb=extra, contextual_emb=ctx.detach())[0]
    assert torch.allclose(l_full, loss.detach(), atol=2e-5)


def test_multitask_head_losses():
    cfg = tiny_hstu(tasks=(("listen_plus", 1, "binary"), ("like", 2, "binary"), ("watch", 0, "regression")))
    head = MultitaskHead(cfg, torch.float32, "cpu")
    T = 7
    g = torch.Generator().manual_seed(0)
    user, item = torch.randn(T, cfg.dim, generator=g), torch.randn(T, cfg.dim, generator=g)
    actions = torch.tensor([0, 1, 2, 3, 4, 5, 6])
    values = torch.rand(T, generator=g)
    losses, preds, labels, w = head(user, item, actions, values)
    assert set(losses) == {"listen_plus", "like", "watch"} and preds.shape == (3, T)
    assert labels[0].tolist() == [0, 1, 0, 1, 0, 1, 0] and labels[1].tolist() == [0, 0, 1, 1, 0, 0, 1]
    logits = head.l2(head.norm(head.l1(user * item))).float().t()
    want = torch.nn.functional.binary_cross_entropy_with_logits(logits[0], labels[0]) * cfg.causal_multitask_weight
    assert torch.allclose(losses["listen_plus"], want, atol=1e-6)
    assert torch.allclose(losses["watch"], ((logits[2] - values) ** 2).mean() * 0.2, atol=1e-6)
    # all-zero supervision weights: the denominator clamps to 1 and the loss is 0
    zero = head(user, item, actions, values, weights=torch.zeros(3, T))[0]
    assert all(float(v) == 0.0 for v in zero.values())


def test_three_stage_pipeline_gives_the_same_losses():
    """Batch N+1's sparse input-dist prepared ahead of step N changes the schedule, not the numbers."""
    from mlperf_training_b200.trainer.hstu import HSTUTrainer
    losses = {}
    for mode in ("plain", "loader", "three_stage"):
        torch.manual_seed(0)
        cfg = tiny_hstu(input_dropout=0.0, linear_dropout=0.0)
        tr = HSTUTrainer(cfg, 300, 6, "cpu", seed=4, data_kw=dict(length_median=10, length_min=3, length_max=30))
        tr.pipelined = mode != "plain"
        tr.pipeline_input_dist = mode == "three_stage"
        losses[mode] = [float(tr.train_step()) for _ in range(5)]
    assert losses["plain"] == losses["loader"] == losses["three_stage"]
    assert losses["plain"][-1] == losses["plain"][-1] and len(set(losses["plain"])) > 1


def test_action_branch_issued_early_is_bit_identical():
    """The action branch computed ahead of the embeddings and handed to forward gives the same loss and gradients."""
    import torch
    from mlperf_training_b200.data.hstu_synth import HSTUSyntheticData
    from mlperf_training_b200.models.hstu import HSTU, HSTUConfig
    cfg = HSTUConfig(layers=2, dim=64, heads=2, d_qk=16, d_v=16, max_seq_len=64, emb_dim=32, mlp_hidden=32, dtype="fp32",
                     input_dropout=0.0, linear_dropout=0.0)
    torch.manual_seed(0)
    model = HSTU(cfg, "cpu", seed=1)
    data = HSTUSyntheticData(1000, 4, seed=0, length_median=20, length_min=4, length_max=60)
    batch = data.batch_at(0, 0)
    emb = torch.randn(batch["rows"], cfg.emb_dim)
    res = []
    for early in (False, True):
        model.zero_grad()
        pre = model.action_branch(batch, batch["rows"]) if early else None
        loss, _, _ = model(batch, emb, action_out=pre)
        loss.backward()
        res.append((loss.detach().clone(), [p.grad.clone() for p in model.parameters() if p.grad is not None]))
    assert torch.equal(res[0][0], res[1][0])
    assert all(torch.equal(a, b) for a, b in zip(res[0][1], res[1][1]))


def _tiny(**kw):
    import torch
    from mlperf_training_b200.data.hstu_synth import HSTUSyntheticData
    from mlperf_training_b200.models.hstu import HSTU, HSTUConfig
    base = dict(layers=3, dim=64, heads=2, d_qk=16, d_v=16, max_seq_len=64, emb_dim=32, mlp_hidden=32, dtype="fp32",
                input_dropout=0.0, linear_dropout=0.0, targets_only_last=False)
    base.update(kw)
    cfg = HSTUConfig(**base)
    torch.manual_seed(0)
    model = HSTU(cfg, "cpu", seed=1)
    data = HSTUSyntheticData(1000, 4, seed=0, length_median=20, length_min=4, length_max=60)
    batch = data.batch_at(0, 0)
    emb = torch.randn(batch["rows"], cfg.emb_dim)
    return cfg, model, batch, emb


def test_stochastic_depth_skips_layers_deterministically():
    import torch
    cfg, model, batch, emb = _tiny(sd_ratio=0.5, sd_seed=7)
    plain_cfg, plain, _, _ = _tiny()
    plain.load_state_dict(model.state_dict())
    rng = torch.get_rng_state()
    draws = [model.skipped_layers(it) for it in range(20)]
    assert torch.equal(rng, torch.get_rng_state())                    # the global generator is untouched
    assert draws == [model.skipped_layers(it) for it in range(20)]    # a function of (seed, layer, forward number)
    assert any(d for d in draws) and any(len(d) < cfg.layers for d in draws)
    model.eval(); plain.eval()
    assert torch.equal(model(batch, emb)[0], plain(batch, emb)[0])    # evaluation never skips
    model.train()
    it = next(i for i, d in enumerate(draws) if d)                    # a forward in which something is skipped
    model.set_extra_state({"sd_iter": it})
    loss = model(batch, emb)[0]
    assert model.get_extra_state()["sd_iter"] == it + 1
    # the same forward with those layers removed by hand
    plain.train()
    kept = [l for i, l in enumerate(plain.layers) if i not in draws[it]]
    plain.layers = torch.nn.ModuleList(kept)
    assert torch.allclose(loss, plain(batch, emb)[0], atol=1e-6)
    full_ratio = _tiny(sd_ratio=1.0)[1]
    assert full_ratio.skipped_layers(3) == [0, 1, 2]


def test_recent_window_layers_leave_old_tokens_untouched():
    import torch
    cfg, model, batch, emb = _tiny(recent_window=8, recent_window_layers=1)
    wide_cfg, wide, _, _ = _tiny(recent_window=4096, recent_window_layers=1)
    plain_cfg, plain, _, _ = _tiny()
    wide.load_state_dict(model.state_dict()); plain.load_state_dict(model.state_dict())
    # a window that covers every sequence changes only the attention's length bound: run the plain model with that bound
    offsets, nt = batch["offsets"], batch["num_targets"]
    total = int(batch["total"])
    lens = (offsets[1:] - offsets[:-1]).long()
    seq = torch.repeat_interleave(torch.arange(lens.numel()), lens)
    col = torch.arange(total) - offsets[:-1].long()[seq]
    x = torch.randn(batch["rows"], cfg.dim)
    layer = model.layers[-1]
    max_t = int(batch.get("max_targets", 0)) or int(nt.max())
    y = model._recent_window_layer(layer, x, offsets, nt, seq, col, total, max_t)
    prefix = (lens - 8 - nt.long()).clamp(min=0)
    old = col < prefix[seq]
    assert old.any() and torch.equal(y[:total][old], x[:total][old])                    # bypassed rows keep their value
    assert not torch.allclose(y[:total][~old], x[:total][~old])
    # the recent rows equal the layer run on a batch made of the windows alone
    keep = ~old
    lens2 = lens - prefix
    off2 = torch.zeros_like(offsets); off2[1:] = torch.cumsum(lens2, 0).to(offsets.dtype)
    n_keep = int(keep.sum())
    rows2 = (n_keep + 127) // 128 * 128
    x2 = torch.zeros(rows2, cfg.dim); x2[:n_keep] = x[:total][keep]
    ref = layer(x2, off2, nt, rows2, max_len=min(cfg.max_seq_len, 8 + max_t))
    assert torch.allclose(y[:total][keep], ref[:n_keep], atol=1e-5)
    # end to end: gradients flow to every layer and the loss is finite
    loss = model(batch, emb)[0]
    loss.backward()
    assert torch.isfinite(loss) and all(p.grad is not None for p in model.layers[-1].parameters())


def test_postprocessor_variants():
    import torch
    for kind in ("timestamp_ln", "ln", "l2"):
        cfg, model, batch, emb = _tiny(postprocessor=kind)
        loss = model(batch, emb)[0]
        loss.backward()
        assert torch.isfinite(loss)


def test_content_encoder_concatenates_and_fills_history_with_dummy_rows():
    import torch
    from mlperf_training_b200.models.hstu import ContentEncoder
    torch.manual_seed(0)
    enc = ContentEncoder(8, additional={"genre": 4}, target_enrich={"rank": 3})
    assert enc.output_dim == 15
    L = 10
    is_target = torch.zeros(L, dtype=torch.bool); is_target[[4, 9]] = True
    item = torch.randn(L, 8)
    pay = {"genre": torch.randn(L, 4), "rank": torch.randn(2, 3)}
    out = enc(item, pay, is_target)
    assert out.shape == (L, 15)
    assert torch.equal(out[:, :8], item) and torch.equal(out[:, 8:12], pay["genre"])
    assert torch.equal(out[4, 12:], pay["rank"][0]) and torch.equal(out[9, 12:], pay["rank"][1])
    assert torch.equal(out[0, 12:], enc.dummy["rank"][0]) and torch.equal(out[8, 12:], enc.dummy["rank"][0])
    out.sum().backward()
    assert enc.dummy["rank"].grad is not None and float(enc.dummy["rank"].grad.sum()) == 8 * 3
    plain = ContentEncoder(8)
    assert plain(item, {}, is_target) is item


def test_interleave_preprocessor_layout_and_forward():
    """Interleaved form: every history event is a content token followed by an action token, a target one content
    token.  The layout helper against a per-sample loop; then a forward whose loss reaches both branches and whose
    targets-only last layer equals the full form."""
    lens = torch.tensor([4, 2, 5])
    nt = torch.tensor([1, 1, 2])
    off = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)])
    seq = torch.repeat_interleave(torch.arange(3), lens)
    col = torch.arange(int(lens.sum())) - off[:-1][seq]
    is_t = col >= (lens - nt)[seq]
    off_i, lens_i, dst_c, h_rows, dst_a = HSTU.interleave_layout(lens, nt, seq, col, is_t)
    want_c, want_a, base = [], [], 0
    for L, T in zip(lens.tolist(), nt.tolist()):
        h = L - T
        want_c += [base + 2 * i for i in range(h)] + [base + 2 * h + j for j in range(T)]
        want_a += [base + 2 * i + 1 for i in range(h)]
        base += 2 * h + T
    assert dst_c.tolist() == want_c and dst_a.tolist() == want_a and off_i.tolist() == [0, 7, 10, 18]
    assert sorted(dst_c.tolist() + dst_a.tolist()) == list(range(18)) and lens_i.tolist() == [7, 3, 8]

    b = _batch(B=4)
    outs = []
    for tol in (False, True):
        cfg = tiny_hstu(preprocessor="interleave", contextual=2, input_dropout=0.0, linear_dropout=0.0, targets_only_last=tol)
        m = HSTU(cfg, "cpu", seed=4)
        g = torch.Generator().manual_seed(2)
        emb = torch.randn(b["rows"], cfg.emb_dim, generator=g)
        emb[b["total"]:] = 0
        ctx = torch.randn(4, 2, cfg.emb_dim, generator=g)
        loss, preds, labels = m(b, emb, contextual_emb=ctx)
        loss.backward()
        assert torch.isfinite(loss) and preds.shape == (4,)
        assert m.content_mlp.l1.weight.grad.abs().sum() > 0 and m.action_mlp.l1.weight.grad.abs().sum() > 0
        outs.append(loss.detach())
    assert torch.allclose(outs[0], outs[1], atol=2e-5)
    # the action of a history event is its own token now: changing one action changes the loss, the sum form's
    # action branch is not part of the content token
    b2 = dict(b, actions=b["actions"].clone())
    b2["actions"][0] ^= 1
    assert not torch.allclose(m(b2, emb, contextual_emb=ctx)[0], outs[1])


def test_parameterized_contextual_mlp_matches_per_sample_matmul():
    from mlperf_training_b200.models.hstu import _ParameterizedMLP
    torch.manual_seed(0)
    mlp = _ParameterizedMLP(12, 6, 8, 5, torch.float32, "cpu")
    with torch.no_grad():
        mlp.norm_w.uniform_(0.5, 1.5)
        mlp.norm_b.uniform_(-0.1, 0.1)
    lens = torch.tensor([3, 1, 4])
    seq = torch.repeat_interleave(torch.arange(3), lens)
    col = torch.cat([torch.arange(int(n)) for n in lens])
    x = torch.randn(16, 6)
    x[8:] = 0
    ctx = torch.randn(3, 12)
    y = mlp(x, seq, col, 3, 4, ctx)
    assert y.shape == (16, 5) and torch.equal(y[8:], torch.zeros(8, 5))
    shared = mlp.compress(ctx)
    for t in range(8):
        s = int(seq[t])
        w = torch.nn.functional.layer_norm(mlp.raw(shared[s:s + 1]).view(6, 5), (6, 5), mlp.norm_w, mlp.norm_b, 1e-5)
        bias = mlp.res2(mlp.res_n(mlp.res1(shared[s:s + 1])))[0]
        assert torch.allclose(y[t], x[t] @ w + bias, atol=1e-5)
    # through the model: the contextual features of a sample steer its own content / action maps only
    b = _batch(B=4)
    cfg = tiny_hstu(contextualized_mlp="parameterized", contextual=2, input_dropout=0.0, linear_dropout=0.0)
    m = HSTU(cfg, "cpu", seed=6)
    g = torch.Generator().manual_seed(3)
    emb = torch.randn(b["rows"], cfg.emb_dim, generator=g)
    ctx = torch.randn(4, 2, cfg.emb_dim, generator=g)
    loss, preds, _ = m(b, emb, contextual_emb=ctx)
    loss.backward()
    assert torch.isfinite(loss) and m.content_mlp.raw.weight.grad.abs().sum() > 0 and m.action_mlp.res2.weight.grad.abs().sum() > 0
    ctx2 = ctx.clone()
    ctx2[2] += 0.5
    changed = (m(b, emb, contextual_emb=ctx2)[1] - preds).abs() > 1e-7
    assert changed.tolist() == [False, False, True, False]
