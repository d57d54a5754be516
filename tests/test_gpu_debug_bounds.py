"""The bounds-reporting debug build: an id outside its table is skipped AND recorded in the status
block (no trap, the context stays usable); the release build skips it silently."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DBG = ROOT / "mlperf_training_b200" / "_b200_kernels_dbg.so"

SCRIPT = r"""
import torch
from mlperf_training_b200.ops import _lib, kernels as K
table = torch.arange(40, dtype=torch.float32, device="cuda").view(5, 8).bfloat16()
ids = torch.tensor([1, 7, 3, -2], device="cuda")            # 7 and -2 are outside the 5-row table
out = K.gather_rows(table, ids)
torch.cuda.synchronize()
st = _lib.status()
print("ROWS", out[0, 0].item(), out[1].abs().sum().item(), out[2, 0].item(), out[3].abs().sum().item())
print("STATUS", st["code"], st["where"], st["count"])
_lib.reset_status()
ok = K.gather_rows(table, torch.tensor([0, 4], device="cuda"))
torch.cuda.synchronize()
print("AFTER", _lib.status()["code"], ok[1, 0].item())
"""


def _run(lib: str | None):
    env = dict(os.environ, PYTHONPATH=str(ROOT))
    if lib:
        env["B200_KERNELS_LIB"] = lib
    r = subprocess.run([sys.executable, "-c", SCRIPT], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout


def test_debug_build_reports_out_of_range_ids_and_release_build_skips_them():
    if not DBG.exists():
        from mlperf_training_b200.csrc.build import build
        build(debug_bounds=True)
    rel = _run(None)
    assert "ROWS 8.0 0.0 24.0 0.0" in rel and "STATUS 0 " in rel          # skipped, nothing recorded
    dbg = _run(str(DBG))
    assert "ROWS 8.0 0.0 24.0 0.0" in dbg                                  # same result: the access is skipped, not trapped
    assert "STATUS 3 401 2" in dbg                                         # B200_ERR_BOUNDS, gather_rows tag, two bad ids
    assert "AFTER 0 32.0" in dbg                                           # the context is fine afterwards
