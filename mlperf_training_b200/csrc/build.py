"""Builds every CUDA source of this directory for sm_100a into one in-tree shared library.

The library (``mlperf_training_b200/_b200_kernels.so``) is loaded with ctypes by
``mlperf_training_b200.ops._lib``; it links the CUDA runtime statically and fetches the one
driver entry point it needs (tensor-map encoding) through the runtime, so it builds on a
machine without a GPU or driver.  Objects are cached by source/flag hash under
``csrc/build/``.

The reference builds its native kernels at run time with hipcc into a /tmp cache keyed by
source + flags + arch (generative_recommenders/ops/hip/k512_fp8_gemm.py:708-805); here the
build is an explicit ahead-of-time step so that the binary travels with the tree.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
LIB_NAME = "_b200_kernels.so"
LIB_PATH = PKG / LIB_NAME

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build the sm_100a kernels")
    return nvcc


def _digest(path: Path, extra: str) -> str:
    h = hashlib.sha256()
    h.update(path.read_bytes())
    for hdr in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(hdr.read_bytes())
    h.update(extra.encode())
    return h.hexdigest()[:16]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


DEBUG_LIB_NAME = "_b200_kernels_dbg.so"


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False, debug_bounds: bool = False) -> Path:
    """Compile all ``*.cu`` files and link the shared library.  Returns its path.  ``debug_bounds`` builds
    the bounds-reporting variant (``-DB200_DEBUG_BOUNDS``) into ``_b200_kernels_dbg.so``; point
    ``B200_KERNELS_LIB`` at it to run a program over it."""
    nvcc = _nvcc()
    obj_dir = CSRC / ("build_dbg" if debug_bounds else "build")
    obj_dir.mkdir(exist_ok=True)
    lib_path = PKG / DEBUG_LIB_NAME if debug_bounds else LIB_PATH
    flags = list(NVCC_FLAGS) + os.environ.get("B200_NVCC_EXTRA", "").split()      # tuning macros
    if debug_bounds:
        flags.append("-DB200_DEBUG_BOUNDS")
    if ptxas_info:
        flags += ["-Xptxas", "-v"]
    flag_key = " ".join(flags)

    def compile_one(src: Path) -> tuple[Path, bool, str]:
        obj = obj_dir / f"{src.stem}.{_digest(src, flag_key)}.o"
        if obj.exists() and not force:
            return obj, False, ""
        for old in obj_dir.glob(f"{src.stem}.*.o"):
            old.unlink()
        cmd = [nvcc, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        return obj, True, res.stderr

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        results = list(ex.map(compile_one, sources()))
    objs = [r[0] for r in results]
    rebuilt = any(r[1] for r in results)
    if verbose or ptxas_info:
        for r in results:
            if r[2]:
                print(r[2], file=sys.stderr)
    if rebuilt or not lib_path.exists() or force:
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
               "-o", str(lib_path), *[str(o) for o in objs]]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return lib_path


if __name__ == "__main__":
    path = build(verbose=True, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv,
                 debug_bounds="--debug-bounds" in sys.argv)
    print(path)
