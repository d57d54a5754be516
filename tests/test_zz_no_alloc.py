"""The allocation-free sum-of-squares entry point, called through its exported C symbol, against
the regular entry point (collected last by name so it also runs after every other GPU test)."""
import ctypes

import pytest
import torch

from mlperf_training_b200.ops import _lib
from mlperf_training_b200.ops import kernels as K

pytestmark = pytest.mark.gpu


def _entry():
    lib = _lib.load()
    fn = lib.b200_sumsq_static
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    lib.b200_sumsq_static_max_elems.restype = ctypes.c_longlong
    lib.b200_last_error.restype = ctypes.c_char_p
    return lib, fn


def test_static_scratch_sumsq_matches_regular_entry_twice():
    lib, fn = _entry()
    torch.manual_seed(0)
    stream = _lib.stream_ptr()
    cases = [torch.randn(40_000_037, device="cuda"), torch.randn(1_000_003, device="cuda").bfloat16()]
    for x in cases:                                     # two calls in a row share the scratch array
        got = torch.zeros(1, device="cuda")
        want = torch.zeros(1, device="cuda")
        rc = fn(x.data_ptr(), x.numel(), int(x.dtype == torch.bfloat16), got.data_ptr(), 0, stream)
        assert rc == 0, lib.b200_last_error()
        K.sumsq(x, want)
        exact = (x.double() ** 2).sum().item()
        assert abs(got.item() - want.item()) <= 1e-5 * abs(exact)
        assert abs(got.item() - exact) <= 1e-5 * abs(exact)
    # accumulate on top of the previous value
    x = cases[1]
    acc = torch.full((1,), 5.0, device="cuda")
    assert fn(x.data_ptr(), x.numel(), 1, acc.data_ptr(), 1, stream) == 0
    assert abs(acc.item() - 5.0 - (x.double() ** 2).sum().item()) <= 1e-5 * (x.double() ** 2).sum().item()
    _lib.check_status("sumsq_static")


def test_static_scratch_sumsq_call_path_allocates_nothing():
    """After the set-up call, a call changes neither torch's allocator figures nor the driver's count
    of free device memory: the property that callers without an allocator rely on."""
    lib, fn = _entry()
    x = torch.randn(3_000_001, device="cuda")
    out = torch.zeros(1, device="cuda")
    stream = _lib.stream_ptr()
    assert fn(x.data_ptr(), x.numel(), 0, out.data_ptr(), 0, stream) == 0          # set-up call for this device
    torch.cuda.synchronize()
    before = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved(), torch.cuda.mem_get_info()[0])
    for _ in range(3):
        assert fn(x.data_ptr(), x.numel(), 0, out.data_ptr(), 0, stream) == 0
    torch.cuda.synchronize()
    after = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved(), torch.cuda.mem_get_info()[0])
    assert after == before, (before, after)
    assert abs(out.item() - (x.double() ** 2).sum().item()) <= 1e-5 * (x.double() ** 2).sum().item()


def test_static_scratch_sumsq_rejects_oversize():
    lib, fn = _entry()
    x = torch.zeros(8, device="cuda")
    out = torch.zeros(1, device="cuda")
    too_many = lib.b200_sumsq_static_max_elems() + 1
    rc = fn(x.data_ptr(), too_many, 0, out.data_ptr(), 0, _lib.stream_ptr())     # refused before any launch
    assert rc != 0
    assert b"outside" in lib.b200_last_error()
    assert out.item() == 0.0
