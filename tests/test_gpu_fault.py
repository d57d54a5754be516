"""A device-side wait that runs out returns an error status the host can read; the context stays
usable (no trap, no hang: the wait is bounded to 50 ms and nothing ever sets the flag)."""
import pytest
import torch

from mlperf_training_b200.ops import _lib
from mlperf_training_b200.ops import kernels as K

pytestmark = pytest.mark.gpu


def test_bounded_wait_reports_timeout_and_context_survives():
    _lib.reset_status()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    res = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    _lib.call("b200_flag_wait_probe", _lib.ptr(flag), 1, 50_000_000, _lib.ptr(res), _lib.stream_ptr())
    torch.cuda.synchronize()
    st = _lib.status()
    assert st["code"] == 2 and st["where"] == 99 and int(res.item()) == 0
    with pytest.raises(RuntimeError, match="flag wait timed out"):
        _lib.check_status("probe")
    assert _lib.status()["code"] == 0                      # check_status cleared it
    # a flag that IS set lets the wait through
    flag.fill_(3)
    _lib.call("b200_flag_wait_probe", _lib.ptr(flag), 2, 50_000_000, _lib.ptr(res), _lib.stream_ptr())
    torch.cuda.synchronize()
    assert int(res.item()) == 1 and _lib.status()["code"] == 0
    # the context still runs kernels
    a = torch.randn(256, 128, device="cuda").bfloat16()
    b = torch.randn(128, 128, device="cuda").bfloat16()
    out = K.gemm(a, b)
    assert torch.allclose(out.float(), a.float() @ b.float().t(), atol=0.5, rtol=5e-2)
