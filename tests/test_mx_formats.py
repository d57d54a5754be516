"""The narrow members of the micro-scaled family (MXFP6, MXFP4, A6W4) carried as e4m3 codes, stochastic rounding,
the Hadamard transform of the weight-gradient operands, and weight de-oscillation."""
import torch

from mlperf_training_b200.ops import functional as F
from mlperf_training_b200.ops import linear as L
from mlperf_training_b200.ops import mxfp8 as MX
from mlperf_training_b200.ops.recipe import DeoscConfig, Deoscillator
from mlperf_training_b200.parallel.engine import OptimConfig, ZeroEngine


def test_element_grids_and_container_exactness():
    grid = lambda fmt, hi: sorted(set(MX.round_to_format(torch.linspace(0, hi, 100001), fmt).tolist()))
    assert grid("e2m1", 8.0) == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    g6 = grid("e2m3", 9.0)
    assert len(g6) == 32 and g6[1] == 0.125 and g6[-1] == 7.5
    g32 = grid("e3m2", 40.0)
    assert len(g32) == 32 and g32[1] == 0.0625 and g32[-1] == 28.0
    # e4m3 through the generic routine equals the hardware cast, ties to even included
    y = torch.cat([torch.randn(20000) * 40, torch.tensor([0.0, 2.5 * 2 ** -9, 17.0, 19.0, 500.0, -500.0])])
    assert torch.equal(MX.round_to_format(y, "e4m3"), y.clamp(-448, 448).to(torch.float8_e4m3fn).float())
    assert MX.round_to_format(torch.tensor([2.5, 3.5, 0.25, 0.75]), "e2m1").tolist() == [2.0, 4.0, 0.0, 1.0]   # ties to even
    # every value of the narrow formats is an e4m3 value: the container holds it exactly
    for fmt in ("e2m1", "e2m3", "e3m2"):
        v = torch.tensor(grid(fmt, 40.0))
        assert torch.equal(v.to(torch.float8_e4m3fn).float(), v)
    # an operand: codes decode to grid values times the block's power-of-two scale; the block maximum fits the format
    x = torch.randn(128, 96) * torch.logspace(-3, 2, 96)[None, :]
    op = MX.quantize(x, row_tile=128, fmt="e2m1")[0]
    codes = op.q.view(torch.float8_e4m3fn).float()
    assert set(codes.abs().unique().tolist()) <= {0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0}
    d = MX.dequantize(op)
    blocks = x.view(128, 3, 32).abs().amax(-1)
    assert ((d - x).view(128, 3, 32).abs().amax(-1) <= blocks * 0.26 + 1e-12).all()       # half a grid step of the top binade
    row, col = MX.quantize(x, row_tile=128, col_tile=128, fmt="e2m3", col_fmt="e2m1")
    assert col.rows == 96 and col.k == 128 and (MX.dequantize(row) - x).abs().mean() < (MX.dequantize(col).t() - x).abs().mean()


def test_stochastic_rounding_is_unbiased_and_on_the_grid():
    torch.manual_seed(0)
    y = torch.full((400000,), 2.3)
    r = MX.round_to_format(y, "e2m1", stochastic=True)
    assert set(r.unique().tolist()) == {2.0, 3.0} and abs(float(r.mean()) - 2.3) < 5e-3
    r = MX.round_to_format(torch.full((400000,), -0.2), "e2m1", stochastic=True)
    assert set(r.unique().tolist()) == {-0.5, 0.0} and abs(float(r.mean()) + 0.2) < 5e-3
    assert float(MX.round_to_format(torch.tensor([7.0]), "e2m1", stochastic=True)) == 6.0          # saturates


def test_hadamard_rows_keeps_the_product():
    torch.manual_seed(1)
    a, b = torch.randn(64, 24), torch.randn(64, 40)
    assert torch.allclose(L.hadamard_rows(a, 16).t() @ L.hadamard_rows(b, 16), a.t() @ b, atol=1e-4)
    # an outlier row is spread over its block: the largest magnitude drops
    a[5] *= 50
    assert L.hadamard_rows(a, 16).abs().max() < 0.5 * a.abs().max()


def test_recipes_order_by_error_and_narrow_weights_are_cached_per_format():
    torch.manual_seed(0)
    x = torch.randn(256, 256)
    w = torch.nn.Parameter(torch.randn(128, 256) * 0.05)
    g = torch.randn(256, 128)
    ref_y, ref_dx, ref_dw = x @ w.t(), g @ w.detach(), g.t() @ x
    err = {}
    for prec in ("mxfp8", "mxfp6", "a6w4", "mxfp4", "mxfp8_fwd_mxfp4_bwd"):
        xx = x.clone().requires_grad_(True)
        w.grad = None
        y = F.linear(xx, w, None, None, prec)
        y.backward(g)
        rel = lambda a, b: float((a - b).norm() / b.norm())
        err[prec] = (rel(y.detach(), ref_y.detach()), rel(xx.grad, ref_dx), rel(w.grad, ref_dw))
    assert err["mxfp8"][0] < err["mxfp6"][0] * 1.2 < err["a6w4"][0] < err["mxfp4"][0] < 0.25
    assert err["mxfp8"][2] < err["mxfp6"][2] < err["mxfp4"][2] < 0.3
    assert abs(err["mxfp8_fwd_mxfp4_bwd"][0] - err["mxfp8"][0]) < 1e-6 and err["mxfp8_fwd_mxfp4_bwd"][1] > 2 * err["mxfp8"][1]
    # the cache key carries the formats: switching recipes re-quantises the weight
    F.linear(x, w, None, None, "mxfp4")
    k4 = w._mx_cache[0]
    F.linear(x, w, None, None, "mxfp8")
    assert k4[1:] == ("e2m1", "e2m1") and w._mx_cache[0][1:] == ("e4m3", "e4m3")
    # the gradient operand is rounded stochastically (unbiased): averaging draws removes its share of the error; what
    # stays is the deterministic rounding of the saved activation
    acc = torch.zeros_like(ref_dw)
    for i in range(24):
        torch.manual_seed(100 + i)
        w.grad = None
        F.linear(x.clone().requires_grad_(True), w, None, None, "mxfp4").backward(g)
        acc += w.grad / 24
    assert float((acc - ref_dw).norm() / ref_dw.norm()) < 0.7 * err["mxfp4"][2]


def test_deoscillator_snaps_flipping_weights_only():
    """A weight dithering across a rounding boundary of the 4-bit grid is set to its grid value at the period end; a
    weight that travels steadily across the grid and a weight at rest are left alone."""
    torch.manual_seed(0)
    lin = torch.nn.Linear(128, 128, bias=False)
    w = lin.weight
    with torch.no_grad():
        w.fill_(0.1)
        w[:, 0::32] = 6.0                 # fixes every block's scale at 1: grid 0, .5, 1, 1.5, 2, 3, 4, 6
        w[0, 1] = 1.26                    # boundary between 1 and 1.5 is 1.25: will dither
        w[0, 2] = 0.6                     # will walk upwards across several grid values
    eng = ZeroEngine(lin, OptimConfig(lr=1e-3, weight_decay=0.0, clip_grad=0.0))
    w = lin.weight
    F.linear(torch.randn(128, 128), w, None, None, "mxfp4")             # a micro-scaled linear has quantised it: tracked
    de = Deoscillator(eng, DeoscConfig(enabled=True, start_step=2, period=10, ratio=4.0))
    snapped = []
    for step in range(12):
        with torch.no_grad():
            w[0, 1] = 1.26 if step % 2 == 0 else 1.24
            w[0, 2] = 0.6 + 0.35 * step
        assert de.after_step(step, "mxfp8") == 0                       # idle under 8-bit weights
        snapped.append(de.after_step(step, "mxfp4"))
    assert snapped == [0] * 11 + [1] and de.snapped == 1 and de.history == [(11, 1)]
    assert float(w[0, 1]) in (1.0, 1.5) and abs(float(w[0, 2]) - (0.6 + 0.35 * 11)) < 1e-6 and abs(float(w[1, 1]) - 0.1) < 1e-7
    st = de.state[id(eng.buckets[0])]
    assert int(st["flips"].sum()) == 0                                 # a new period starts clean


def test_run_loop_switches_recipes_and_deoscillates():
    """MXFP4 with de-oscillation for three steps, then MXFP8: the run differs from a pure MXFP8 run before the switch
    and the de-oscillator reports a period end."""
    import io

    from mlperf_training_b200.trainer.loop import run
    tiny = dict(n_layers=2, hidden=128, n_heads=2, n_kv_heads=2, head_dim=64, ffn_hidden=256, vocab_size=256, seq_len=128,
                dtype="fp32", precision="mxfp8")
    base = dict(model=tiny, global_batch=2, micro_batch=2, train_iters=5, lr=2e-3, lr_warmup_iters=1, clip_grad=1.0)
    plain = run(dict(base), device="cpu", stream=io.StringIO())
    sw = run(dict(base, precision_schedule={"initial": "mxfp4", "switch_step": 3, "final": "mxfp8",
                                            "deosc": {"enabled": True, "start_step": 0, "period": 2, "ratio": 1.0}}),
             device="cpu", stream=io.StringIO())
    assert sw["precision_log"] == [(0, "mxfp4"), (3, "mxfp8")]
    assert [s for s, _ in sw["deosc_history"]] == [1]                  # one full period (steps 0-1) under 4-bit weights, then idle
    assert all(l == l for l in sw["losses"]) and abs(sw["losses"][0] - plain["losses"][0]) > 1e-4
    assert abs(sw["losses"][0] - plain["losses"][0]) < 0.2             # 4-bit forward: close, not equal


def test_deoscillator_tracks_stacked_expert_weights():
    from mlperf_training_b200.ops import moe_ops as M

    class Experts(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.w1 = torch.nn.Parameter((torch.randn(2, 384, 192) * 0.05).bfloat16())
            self.w2 = torch.nn.Parameter((torch.randn(2, 192, 192) * 0.05).bfloat16())
    torch.manual_seed(0)
    m = Experts()
    eng = ZeroEngine(m, OptimConfig(lr=1e-3, weight_decay=0.0, clip_grad=0.0))
    x = torch.randn(64, 192).bfloat16()
    idx, w, counts = M.router_topk(torch.randn(64, 2), 1)
    M.moe_experts(x, idx, w, counts, m.w1, m.w2, "mxfp4")              # the grouped MLP has quantised the stacks
    de = Deoscillator(eng, DeoscConfig(enabled=True, start_step=0, period=6, ratio=2.0))
    with torch.no_grad():
        m.w1[1, 5, :32] = 0.1
        m.w1[1, 5, 0] = 6.0
    for step in range(6):
        with torch.no_grad():
            m.w1[1, 5, 3] = 1.27 if step % 2 == 0 else 1.23
        n = de.after_step(step, "mxfp4")
    assert n == 1 and float(m.w1[1, 5, 3]) in (1.0, 1.5)
    assert eng.buckets[0].master is None or float(eng.buckets[0].master.max()) <= 6.0


def test_flux_loop_switches_forward_precision():
    """The diffusion run loop: forward in A6W4 until the switch step, then 8-bit forward with a 4-bit backward; the
    switch is logged and changes the losses against a run that never switches."""
    import io

    from mlperf_training_b200.trainer.flux import run
    base = dict(model=dict(preset="tiny-mmdit"), global_batch=8, train_iters=4, lr=1e-3, prompt_dropout=0.0)
    spec = {"initial": "a6w4", "switch_step": 2, "final": "mxfp8_fwd_mxfp4_bwd",
            "deosc": {"enabled": True, "start_step": 0, "period": 2, "ratio": 1.0}}
    buf = io.StringIO()
    import contextlib
    with contextlib.redirect_stdout(buf):
        sw = run(dict(base, precision_schedule=spec), device="cpu", stream=io.StringIO())
        stay = run(dict(base, precision_schedule={"initial": "a6w4"}), device="cpu", stream=io.StringIO())
    text = buf.getvalue()
    assert "step 0: linears run in a6w4" in text and "step 2: linears run in mxfp8_fwd_mxfp4_bwd" in text
    assert "deosc: on" in text
    assert all(l == l for l in sw["losses"]) and sw["losses"][:2] == stay["losses"][:2] and sw["losses"][2] != stay["losses"][2]


def test_deoscillator_state_survives_a_resume(tmp_path):
    """A run under 4-bit weights that exits in the middle of a de-oscillation period and resumes ends on the losses of
    the uninterrupted run: flip counts travel with the optimizer shard."""
    import io

    import pytest

    from mlperf_training_b200.trainer.loop import run
    tiny = dict(n_layers=2, hidden=128, n_heads=2, n_kv_heads=2, head_dim=64, ffn_hidden=256, vocab_size=256, seq_len=128,
                dtype="fp32", precision="mxfp4")
    spec = {"initial": "mxfp4", "deosc": {"enabled": True, "start_step": 0, "period": 4, "ratio": 0.5}}
    base = dict(model=tiny, global_batch=2, micro_batch=2, train_iters=6, lr=5e-3, lr_warmup_iters=1, clip_grad=1.0,
                precision_schedule=spec)
    torch.manual_seed(0)
    ref = run(dict(base), device="cpu", stream=io.StringIO())
    assert [s for s, _ in ref["deosc_history"]] == [3]
    e = dict(base, checkpoint_dir=str(tmp_path / "ck"), die_at_step=2)
    torch.manual_seed(0)
    with pytest.raises(SystemExit):
        run(dict(e), device="cpu", stream=io.StringIO())
    out = run(dict(e, die_at_step=0), device="cpu", stream=io.StringIO())
    assert out["steps"] == 4 and out["deosc_history"] == ref["deosc_history"]         # same count snapped at the same step
    assert max(abs(a - b) for a, b in zip(out["losses"], ref["losses"][2:])) < 1e-5


def test_deoscillation_keeps_replicas_identical_gloo():
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=root)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29679",
                        os.path.join(root, "tests", "multi", "deosc_worker.py")], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("ok=True") == 2
