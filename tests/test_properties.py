"""Property-based checks (hypothesis) of host-side arithmetic: mesh group construction, pipeline layer split, zig-zag
chunking, the interleaved token layout, element-format rounding, sort / segment-sum oracles, embedding placement."""
import torch
from hypothesis import given, settings, strategies as st

from mlperf_training_b200.models.hstu import HSTU
from mlperf_training_b200.ops import mxfp8 as MX
from mlperf_training_b200.ops import sort as S
from mlperf_training_b200.parallel.context import zigzag_chunk, zigzag_unchunk
from mlperf_training_b200.parallel.embedding_collection import TableConfig, plan_tables
from mlperf_training_b200.parallel.mesh import MeshSpec, coords, group_ranks
from mlperf_training_b200.parallel.pipeline import stage_layers

FAST = settings(max_examples=40, deadline=None)


@FAST
@given(tp=st.sampled_from([1, 2, 4]), cp=st.sampled_from([1, 2]), pp=st.sampled_from([1, 2, 3]), dp=st.sampled_from([1, 2, 4]),
       ep=st.sampled_from([1, 2, 4]), rep=st.sampled_from([1, 2]))
def test_mesh_groups_partition_the_world(tp, cp, pp, dp, ep, rep):
    if dp % ep or dp % rep:
        return
    spec = MeshSpec(tp=tp, pp=pp, cp=cp, ep=ep, dp_replicate=rep)
    world = tp * cp * pp * dp
    groups = group_ranks(spec, world)
    sizes = {"tp": tp, "cp": cp, "pp": pp, "dp": dp, "ep": ep, "edp": dp // ep, "dp_shard": dp // rep, "dp_replicate": rep,
             "dp_cp": dp * cp, "edp_cp": dp // ep * cp}
    for dim, lists in groups.items():
        flat = sorted(r for g in lists for r in g)
        assert flat == list(range(world)), dim                          # every rank in exactly one group of the dimension
        assert all(len(g) == sizes[dim] for g in lists), dim
    for r in range(world):
        c = coords(r, spec, world)
        assert 0 <= c["tp"] < tp and 0 <= c["cp"] < cp and 0 <= c["pp"] < pp and 0 <= c["dp"] < dp
    # ranks of a tensor-parallel group are neighbours; pipeline stages are the outermost dimension
    assert all(g == list(range(g[0], g[0] + tp)) for g in groups["tp"])
    assert all(b - a == world // pp for g in groups["pp"] for a, b in zip(g, g[1:]))
    # an expert-parallel group and an expert-data-parallel group meet in exactly one rank
    for g in groups["ep"]:
        for h in groups["edp"]:
            if set(g) & set(h):
                assert len(set(g) & set(h)) == 1


@FAST
@given(n_layers=st.integers(1, 96), n_stages=st.integers(1, 12))
def test_stage_layers_cover_the_model_evenly(n_layers, n_stages):
    if n_stages > n_layers:
        return
    parts = [list(stage_layers(n_layers, n_stages, s)) for s in range(n_stages)]
    assert [i for p in parts for i in p] == list(range(n_layers))
    assert max(map(len, parts)) - min(map(len, parts)) <= 1 and sorted(map(len, parts), reverse=True) == list(map(len, parts))


@FAST
@given(world=st.integers(1, 6), c=st.integers(1, 5), width=st.integers(1, 3))
def test_zigzag_chunks_invert_and_balance(world, c, width):
    t = torch.arange(2 * world * c * width).view(1, 2 * world * c, width)
    pieces = [zigzag_chunk(t, world, r) for r in range(world)]
    assert torch.equal(zigzag_unchunk(pieces), t)
    # causal work of a rank = sum of the positions it holds (+1): equal for every rank
    work = [int((p[0, :, 0] // width + 1).sum()) for p in pieces]
    assert len(set(work)) == 1


@FAST
@given(data=st.data())
def test_interleave_layout_is_a_bijection(data):
    B = data.draw(st.integers(1, 6))
    nt = torch.tensor([data.draw(st.integers(0, 3)) for _ in range(B)])
    lens = torch.tensor([int(nt[i]) + data.draw(st.integers(1, 9)) for i in range(B)])
    off = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)])
    seq = torch.repeat_interleave(torch.arange(B), lens)
    col = torch.arange(int(lens.sum())) - off[:-1][seq]
    is_t = col >= (lens - nt)[seq]
    off_i, lens_i, dst_c, h_rows, dst_a = HSTU.interleave_layout(lens, nt, seq, col, is_t)
    total = int(2 * lens.sum() - nt.sum())
    assert sorted(dst_c.tolist() + dst_a.tolist()) == list(range(total)) and int(off_i[-1]) == total
    assert torch.equal(lens_i, 2 * (lens - nt) + nt)
    # inside a sample: content precedes its action, events keep their order, targets come last
    for b in range(B):
        rows = dst_c[seq == b]
        assert torch.equal(rows, rows.sort().values) and int(rows[0]) == int(off_i[b])
    assert torch.equal(dst_a, dst_c[h_rows] + 1)


@FAST
@given(fmt=st.sampled_from(["e2m1", "e2m3", "e3m2", "e4m3"]), seed=st.integers(0, 10**6), scale=st.floats(1e-3, 1e3))
def test_round_to_format_properties(fmt, seed, scale):
    g = torch.Generator().manual_seed(seed)
    y = torch.randn(512, generator=g) * scale
    r = MX.round_to_format(y, fmt)
    m_bits, e_min, v_max = MX.ELEMENT_FORMATS[fmt]
    assert torch.equal(MX.round_to_format(r, fmt), r)                    # idempotent: results are on the grid
    assert torch.equal(MX.round_to_format(-y, fmt), -r)                  # odd
    assert float(r.abs().max()) <= v_max
    inside = y.abs() <= v_max
    # nearest: the error is at most half the spacing at that magnitude
    _, ex = torch.frexp(y.abs().clamp(min=1e-30))
    half = torch.exp2((ex - 1).clamp(min=e_min).float() - m_bits) / 2
    assert bool(((r - y).abs()[inside] <= half[inside] * (1 + 1e-6)).all())
    order = torch.argsort(y)
    assert bool((r[order][1:] >= r[order][:-1]).all())                   # monotone
    assert torch.equal(r.to(torch.float8_e4m3fn).float(), r)             # an e4m3 value: the container is exact


@FAST
@given(n=st.integers(1, 300), hi=st.integers(1, 50), d=st.sampled_from([1, 4, 8]), seed=st.integers(0, 10**6))
def test_sort_unique_and_segment_sum_oracle(n, hi, d, seed):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, hi, (n,), generator=g)
    s = S.sort_unique(ids, S.key_bits_for(hi))
    cnt = s.n_unique()
    assert torch.equal(s.keys, ids[s.perm]) and torch.equal(s.uniq[:cnt], torch.unique(ids))
    assert torch.equal(s.uniq[s.inverse], ids)
    assert int(s.seg[cnt]) == n and bool((s.seg[1:cnt + 1] > s.seg[:cnt]).all())
    # stable: equal ids keep their original order
    same = s.keys[1:] == s.keys[:-1]
    assert bool((s.perm[1:][same] > s.perm[:-1][same]).all())
    src = torch.randn(n, d, generator=g)
    out = S.segment_sum(src, s)
    want = torch.zeros(cnt, d).index_add_(0, s.inverse, src)
    assert torch.allclose(out[:cnt], want, atol=1e-5) and float(out[cnt:].abs().sum()) == 0


@FAST
@given(world=st.sampled_from([1, 2, 4, 8]), sizes=st.lists(st.integers(1, 2000), min_size=1, max_size=9), cut=st.integers(1, 3000))
def test_embedding_plan_places_every_table_once(world, sizes, cut):
    tabs = [TableConfig(f"t{i}", rows, 64, (f"f{i}",)) for i, rows in enumerate(sizes)]
    plan = plan_tables(tabs, world, row_wise_min_bytes=cut * 128)
    assert set(plan) == {t.name for t in tabs}
    load = [0] * world
    for t in tabs:
        kind, owner = plan[t.name]
        if world == 1:
            assert kind == "row_wise"
        elif t.bytes() >= cut * 128:
            assert (kind, owner) == ("row_wise", None)
        else:
            assert kind == "table_wise" and 0 <= owner < world
            load[owner] += t.bytes()
    small = sorted((t.bytes() for t in tabs if world > 1 and t.bytes() < cut * 128), reverse=True)
    if small:
        assert max(load) - min(load) <= small[0]                        # greedy by size: ranks differ by at most the largest table


@settings(max_examples=15, deadline=None)
@given(seed=st.integers(0, 1000), seq=st.sampled_from([8, 16, 33]), n_docs=st.integers(1, 12), world=st.sampled_from([1, 2, 4]))
def test_blended_token_dataset_properties(tmp_path_factory, seed, seq, n_docs, world):
    import numpy as np
    from mlperf_training_b200.data.indexed import GPTSampleDataset, write_indexed_dataset
    root = tmp_path_factory.mktemp("idx")
    rng = np.random.default_rng(seed)
    big = [rng.integers(0, 1000, size=int(rng.integers(seq, 6 * seq))).astype(np.int32) for _ in range(n_docs + 3)]
    tiny = [np.arange(3, dtype=np.int32)]                                     # shorter than one sample
    write_indexed_dataset(str(root / "a"), big)
    write_indexed_dataset(str(root / "b"), tiny)
    if sum(len(d) for d in big) <= seq:
        return
    ds = GPTSampleDataset([str(root / "a"), str(root / "b")], [0.5, 0.5], seq, seed=seed)
    stream = np.concatenate(big)
    assert len(ds) == (len(stream) - 1) // seq and set(ds.order_set.tolist()) == {0}     # the short prefix is never drawn
    seen = set()
    for i in range(len(ds)):
        s = ds.sample(i)
        j = int(ds.order_idx[i])
        assert s.shape == (seq + 1,) and np.array_equal(s, stream[j * seq:j * seq + seq + 1])
        seen.add(j)
    assert seen == set(range(len(ds)))                                       # an epoch visits every window once
    again = GPTSampleDataset([str(root / "a"), str(root / "b")], [0.5, 0.5], seq, seed=seed)
    assert np.array_equal(again.order_idx, ds.order_idx)                     # a pure function of the seed
    # the ranks of a step read consecutive, disjoint samples
    got = [ds.batch(3, r, world, 2) for r in range(world)]
    want = [ds.sample((3 * world + r) * 2 + k) for r in range(world) for k in range(2)]
    assert np.array_equal(np.concatenate([g.numpy() for g in got]), np.stack(want))


@settings(max_examples=8, deadline=None)
@given(seed=st.integers(0, 1000), world=st.sampled_from([1, 2, 3]), batch=st.sampled_from([2, 4]), max_history=st.sampled_from([12, 30]))
def test_event_store_stream_properties(tmp_path_factory, seed, world, batch, max_history):
    import numpy as np
    from mlperf_training_b200.data.yambda import EventStoreDataset, write_synthetic_event_store
    root = str(tmp_path_factory.mktemp("store"))
    write_synthetic_event_store(root, 60, 50, 500, days=3, seed=seed)
    kw = dict(max_history=max_history, min_history=4, holdout=0.2, salt=seed)
    train, held = EventStoreDataset(root, batch, split="train", **kw), EventStoreDataset(root, batch, split="eval", **kw)
    users_t, users_e = set(np.asarray(train.user)[train.anchors].tolist()), set(np.asarray(held.user)[held.anchors].tolist())
    assert not users_t & users_e                                             # a user is on one side of the split
    ts = np.asarray(train.ts)
    steps = sum(train.batches_in_window(w, world) for w in range(train.num_windows))
    if steps == 0:
        return
    seen = []
    last_window = -1
    for step in range(steps):
        w = train.window_of_step(step, world)
        assert w >= last_window                                              # windows are walked in time order
        last_window = w
        for rank in range(world):
            anchors = train.step_anchors(step, rank, world)
            b = train.batch_at(step, rank, world=world)
            assert len(anchors) == batch and b["offsets"].numel() == batch + 1 and int(b["offsets"][-1]) == b["total"]
            seen += anchors.tolist()
            for i, a in enumerate(anchors.tolist()):
                lo, hi = int(b["offsets"][i]), int(b["offsets"][i + 1])
                t = b["timestamps"][lo:hi].numpy()
                assert 1 <= hi - lo <= max_history + 1 and t[-1] == ts[a]   # the anchor is the sample's last event
                assert int(np.asarray(train.kind)[a]) == 0                   # anchors are listens
                u = int(np.asarray(train.user)[a])
                assert int(train.uoff[u]) + 4 <= a                           # with at least min_history events before them
    assert len(seen) == len(set(seen))                                       # no anchor is read twice in a pass
    assert b["rows"] % 128 == 0 and b["rows"] >= b["total"]
