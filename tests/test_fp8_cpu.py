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
