"""Per-tensor FP8 recipe on CPU (the eager emulation that the GPU kernels are tested against): delayed
scaling state, linear triple, and a precision schedule whose switch changes the numbers."""
import torch

from mlperf_training_b200.ops import fp8, linear
from mlperf_training_b200.ops import functional as F
from mlperf_training_b200.ops.recipe import PrecisionSchedule, resolve_format


def test_delayed_scale_follows_the_history():
    st = fp8.DelayedScale("e4m3", "cpu", history=2)
    x = torch.randn(256, 256).bfloat16() * 3
    st.prepare(x, epoch=0)                               # first use: the tensor's own maximum
    assert abs(float(st.scale) * float(x.abs().max()) - 448.0) < 1e-3
    row, col = fp8.quantize(x, st, want_row=True, want_col=True)
    assert float(st.amax.view(torch.float32)) == float(x.abs().max())
    err = (fp8.dequantize(row) - x.float()).abs().max() / x.abs().max()
    assert err < 0.07 and torch.equal(fp8.dequantize(col), fp8.dequantize(row).t())
    y = x * 4
    st.prepare(y, epoch=0)                               # same epoch: the factor does not move
    s0 = float(st.scale)
    fp8.quantize(y, st)
    st.prepare(y, epoch=1)                               # next epoch: the collected maximum enters the history
    assert float(st.scale) < s0 and abs(float(st.scale) * float(y.abs().max()) - 448.0) < 1e-2


def test_fp8_linear_triple_is_close_to_bf16_and_differs_from_mxfp8():
    torch.manual_seed(0)
    x = torch.randn(256, 256).bfloat16().requires_grad_(True)
    w = (torch.randn(256, 256) * 0.05).bfloat16().requires_grad_(True)
    dy = torch.randn(256, 256).bfloat16()
    outs = {}
    for pr in ("bf16", "fp8", "mxfp8"):
        xx, ww = x.detach().clone().requires_grad_(True), w.detach().clone().requires_grad_(True)
        y = F.linear(xx, ww, precision=pr)
        y.backward(dy)
        outs[pr] = (y.detach().float(), xx.grad.float(), ww.grad.float())
    for a, b in zip(outs["fp8"], outs["bf16"]):
        assert (a - b).norm() / b.norm() < 0.08
    assert not torch.equal(outs["fp8"][0], outs["mxfp8"][0])      # two recipes, two roundings
    assert resolve_format("fp8_hybrid") == "fp8" and resolve_format("a6w4") == "a6w4"


def test_schedule_switch_changes_the_numbers():
    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.w = torch.nn.Parameter((torch.randn(256, 256) * 0.05).bfloat16())
            self.precision = "bf16"

        def forward(self, x):
            return F.linear(x, self.w, precision=self.precision)

    torch.manual_seed(1)
    m = M()
    x = torch.randn(256, 256).bfloat16()
    sched = PrecisionSchedule.from_spec({"initial": "a6w4", "switch_step": 2, "final": "fp8"})
    ys = []
    for step in range(4):
        sched.apply(m, step)
        ys.append(m(x).float())
    assert torch.equal(ys[0], ys[1]) and torch.equal(ys[2], ys[3])
    assert not torch.equal(ys[1], ys[2])
    assert sched.log == [(0, "a6w4"), (2, "fp8")]


def test_scale_policies_frozen_calibration_and_refresh_cadence():
    """"frozen": the factor follows the first ``history`` epochs and then never moves; ``refresh``: a rolling factor is
    republished only at the end of every window from the maximum collected in it; ``margin`` leaves headroom."""
    old4, old5 = fp8.set_policy("e4m3", mode="frozen", history=2, margin=1.5), fp8.set_policy("e5m2", refresh=3, history=1, margin=8.0)
    try:
        st = fp8.DelayedScale("e4m3", "cpu")
        x = torch.randn(128, 128).bfloat16()
        seen = []
        for epoch, mult in enumerate((1.0, 4.0, 2.0, 100.0, 100.0)):
            st.prepare(x * mult, epoch)
            fp8.quantize(x * mult, st)
            seen.append((float(st.scale), st.frozen))
        amax = float(x.abs().max())
        assert not seen[1][1] and seen[2][1] and seen[2][0] == seen[3][0] == seen[4][0]      # frozen after two calibration epochs
        assert abs(seen[2][0] * amax * 4.0 * 1.5 - 448.0) < 1e-2                            # max of the calibration epochs, margin 1.5
        sd = st.state_dict()
        st2 = fp8.DelayedScale("e4m3", "cpu")
        st2.load_state_dict(sd)
        st2.prepare(x * 1000, 9)
        assert st2.frozen and float(st2.scale) == seen[4][0]                                # a resumed site stays frozen
        g = fp8.DelayedScale("e5m2", "cpu")
        scales = []
        for epoch, mult in enumerate((1.0, 1.0, 8.0, 1.0, 1.0, 1.0, 1.0)):
            g.prepare(x * mult, epoch)
            fp8.quantize(x * mult, g)
            scales.append(float(g.scale))
        # published at epochs 3 and 6 only: the first window's maximum (8 x) rules from epoch 3 on, the second's (1 x) from 6
        assert scales[0] == scales[1] == scales[2] and scales[3] == scales[4] == scales[5] != scales[2]
        assert abs(scales[3] * amax * 8.0 * 8.0 - 57344.0) / 57344.0 < 1e-3 and abs(scales[6] * amax * 8.0 - 57344.0) / 57344.0 < 1e-3
    finally:
        fp8.set_policy("e4m3", **old4)
        fp8.set_policy("e5m2", **old5)


def test_hstu_run_with_the_reference_fp8_policy_resumes(tmp_path):
    """HSTU linears in per-tensor FP8 with calibrate-then-freeze factors: the factor state is part of the model's
    checkpoint, so a run that exits after the calibration and resumes continues on the straight run's losses."""
    import io

    import pytest

    from mlperf_training_b200.trainer.hstu import run
    old4, old5 = dict(fp8.SCALE_POLICY["e4m3"]), dict(fp8.SCALE_POLICY["e5m2"])
    try:
        e = dict(batch_per_gpu=32, train_steps=8, dense_lr=2e-3, sparse_lr=0.05, eval_interval_steps=0, num_eval_batches=0,
                 model=dict(layers=1, dim=256, heads=2, d_qk=128, d_v=128, max_seq_len=64, dtype="fp32", precision="fp8",
                            mlp_hidden=128, num_positions=128, num_time_buckets=32, fp8_scale_policy="reference",
                            fp8_calibration_steps=2, input_dropout=0.0, linear_dropout=0.0),
                 embedding=dict(rows=300, dim=128), data=dict(length_median=24, length_min=8, length_max=60))
        ref = run(dict(e), device="cpu", stream=io.StringIO())
        sites = [s for p in ref["trainer"].model.parameters() for s in getattr(p, "_fp8_sites", {}).values()]
        assert sites and all(s.frozen for s in sites if s.fmt == "e4m3") and any(s.fmt == "e5m2" and not s.frozen for s in sites)
        ck = dict(e, checkpoint_dir=str(tmp_path / "ck"), die_at_step=5)
        with pytest.raises(SystemExit):
            run(dict(ck), device="cpu", stream=io.StringIO())
        out = run(dict(ck, die_at_step=0), device="cpu", stream=io.StringIO())
        assert max(abs(a - b) for a, b in zip(out["losses"], ref["losses"][5:])) < 1e-5
    finally:
        fp8.SCALE_POLICY["e4m3"].update(old4)
        fp8.SCALE_POLICY["e5m2"].update(old5)
