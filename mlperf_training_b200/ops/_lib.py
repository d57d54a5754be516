"""ctypes binding of the in-tree sm_100a kernel library (``_b200_kernels.so``).

Every exported launcher has the C ABI ``int f(..., void* stream)`` and returns 0 or an
error code whose text ``b200_last_error()`` gives; ``call`` turns a non-zero code into a
``RuntimeError``.  The same loading style (C ABI + ctypes, fail loudly) is what the
reference uses for its native kernels
(generative_recommenders/ops/hip/k512_fp8_gemm.cu:555-579 and its Python loader).

On a machine with a GPU the library is mandatory: ``require()`` raises if it cannot be
loaded, so GPU runs never fall back silently to eager PyTorch.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent.parent
# B200_KERNELS_LIB selects another build of the library (the bounds-reporting debug build)
LIB_PATH = Path(os.environ["B200_KERNELS_LIB"]) if os.environ.get("B200_KERNELS_LIB") else _PKG / "_b200_kernels.so"

_lib = None
_lock = threading.Lock()
_load_error: str | None = None

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float


def _declare(lib: ctypes.CDLL) -> None:
    lib.b200_last_error.restype = ctypes.c_char_p
    lib.b200_launch_count.restype = c_ll
    lib.b200_launch_count_reset.restype = None
    lib.b200_status_read.argtypes = [ctypes.POINTER(c_int)]
    lib.b200_sm_count.restype = c_int
    P, I, L, F = c_void_p, c_int, c_ll, c_float
    sigs = {
        "b200_gemm_bf16": [P, P, P, I, I, I, L, L, L, I, I, I, I, P, P, L, F, P],
        "b200_norm_fwd": [I, P, P, P, P, P, P, P, P, I, I, F, I, P],
        "b200_norm_bwd": [I, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, P],
        "b200_rope": [P, P, P, P, L, I, L, I, I, I, I, P],
        "b200_swiglu_fwd": [P, P, L, I, P],
        "b200_swiglu_bwd": [P, P, P, L, I, P],
        "b200_gelu_fwd": [P, P, L, P],
        "b200_gelu_bwd": [P, P, P, L, P],
        "b200_gather_rows": [P, P, P, L, I, L, P],
        "b200_scatter_add_rows": [P, P, P, L, I, L, P],
        "b200_add_bf16": [P, P, P, L, P],
        "b200_accum_f32_bf16": [P, P, L, P],
        "b200_cross_entropy": [P, P, P, P, L, L, I, F, I, L, P],
        "b200_sumsq": [P, L, I, P, P, I, P],
        "b200_adamw": [P, I, P, P, I, P, P, L, F, F, F, F, F, I, F, P, F, I, P],
        "b200_adamw_bf16m": [P, I, P, P, I, P, P, L, F, F, F, F, F, I, F, P, F, I, P],
        "b200_attn_fwd": [P, P, P, P, P, P, I, I, I, I, I, I, L, L, L, L, L, L, L, L, F, I, I, P],
        "b200_quant_mxfp8": [P, L, I, I, P, P, I, P, P, I, P],
        "b200_gemm_mxfp8": [P, P, P, P, P, I, I, I, L, L, L, I, I, P, P, L, F, P],
        "b200_router_topk": [P, I, I, I, P, P, P, P],
        "b200_router_plan": [P, P, I, I, I, P, P, I, P, P],
        "b200_permute_rows": [P, P, I, I, I, P, P, P, P],
        "b200_unpermute_sum": [P, P, P, I, I, I, P, P],
        "b200_gemm_grouped_rows": [P, P, P, P, I, I, I, I, L, L, I, I, F, P],
        "b200_gemm_grouped_wgrad": [P, P, P, P, I, I, I, I, L, L, I, I, F, P],
        "b200_gemm_grouped_mx_rows": [P, P, P, P, P, P, I, I, I, I, L, L, L, I, F, P],
        "b200_gemm_grouped_mx_wgrad": [P, P, P, P, P, P, I, I, I, I, L, L, I, I, F, P],
        "b200_zero_reduce_scatter": [P, I, I, L, L, F, P, P, P],
        "b200_zero_adamw_all_gather": [P, I, I, L, L, P, P, P, P, F, F, F, F, F, I, F, P, F, I, P],
        "b200_zero_reduce_scatter_mc": [P, L, L, F, P, I, P, P],
        "b200_mc_all_gather": [P, P, L, P],
        "b200_zero_adamw_all_gather_mc": [P, P, L, P, P, P, P, F, F, F, F, F, I, F, P, F, I, P],
        "b200_quant_fp8": [P, L, I, I, P, I, P, P, P, P],
        "b200_quant_fp8_rows": [P, L, L, I, P, I, P, L, P, P],
        "b200_hstu_attn_fwd_fp8": [P, P, P, P, P, P, I, L, I, I, I, I, L, L, L, L, F, P, P, P, P],
        "b200_gemm_fp8": [P, P, P, I, I, I, L, L, L, I, I, P, P, I, I, P, P, L, F, P],
        "b200_ln_modulate_fwd": [P, P, P, L, P, P, P, I, I, I, F, P],
        "b200_ln_modulate_bwd": [P, P, P, L, P, P, P, P, P, I, I, I, P],
        "b200_gate_residual_fwd": [P, P, P, L, P, I, I, I, P],
        "b200_gate_residual_bwd": [P, P, P, L, P, P, I, I, I, P],
        "b200_sort_ids": [P, P, P, L, I, P, L, P],
        "b200_unique_segments": [P, P, L, P, P, P, P, P, L, P],
        "b200_segment_sum_gather": [P, I, L, P, P, P, L, L, I, P, I, P, P],
        "b200_hstu_attn_fwd": [P, P, P, P, P, P, I, L, I, I, I, I, L, L, L, L, F, P],
        "b200_hstu_gate_cat_fwd": [P, L, P, P, P, P, P, P, I, I, F, F, ctypes.c_ulonglong, P],
        "b200_hstu_gate_cat_bwd": [P, P, L, P, P, P, P, P, P, L, P, P, P, P, I, I, I, F, ctypes.c_ulonglong, P],
        "b200_hstu_attn_bwd": [P, P, P, P, P, P, P, P, P, I, L, I, I, I, I, L, L, L, L, L, L, F, P],
        "b200_scatter_rows_to_peers": [P, P, P, P, L, I, P, I, L, P, P],
        "b200_gather_rows_from_peers": [P, P, P, L, I, P, I, L, P],
        "b200_zero_pad_rows": [P, P, P, I, I, L, P],
        "b200_ep_route": [P, P, I, I, I, I, L, L, P, P, P, P, P, P],
        "b200_unpermute_bwd": [P, P, P, P, L, I, I, P, P, P],
        "b200_zero_dead_tiles": [P, P, I, I, P],
        "b200_quant_swiglu_mxfp8": [P, L, I, I, P, P, I, P, P, I, P],
        "b200_quant_swiglu_bwd_mxfp8": [P, L, P, L, I, I, P, P, I, P, P, I, P],
        "b200_flag_wait_probe": [P, I, L, P, P],
        "b200_gemm_tp_gather": [P, P, P, I, I, I, L, L, L, I, I, I, I, F, I, P, I, I, P, L, I, P, I, I, P, P],
        "b200_gemm_tp_rs": [P, P, I, I, I, L, L, I, I, F, P, P, I, I, P, P, L, P, L, I, P],
        "b200_gemm_tp_gather_pair": [P, P, P, I, I, I, L, L, L, I, I, I, P, P, F, P, I, I, P, L, I, P, I, I, P, P],
        "b200_gemm_tp_rs_pair": [P, P, I, I, I, L, L, I, I, I, P, P, F, P, P, I, I, P, P, L, P, L, I, P],
        "b200_gemm_tp_gather_fp8": [P, P, P, I, I, I, L, L, L, I, I, P, P, I, I, F, I, P, I, I, P, L, I, P, I, I, P, P],
        "b200_gemm_tp_rs_fp8": [P, P, I, I, I, L, L, I, I, P, P, F, P, P, I, I, P, P, L, P, L, I, P],
        "b200_gather_rows_to_peers": [P, L, P, P, L, I, I, P, P, P],
        "b200_rowwise_adagrad": [P, P, P, P, L, I, F, F, L, P],
        "b200_segment_sum_rows": [P, P, L, I, P, P],
        "b200_attn_delta": [P, P, P, I, I, I, I, L, L, L, L, P],
        "b200_attn_bwd": [P] * 9 + [I] * 6 + [L] * 12 + [F, I, I, P],
    }
    for name, argtypes in sigs.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue
        fn.argtypes = argtypes
        fn.restype = c_int
    lib.b200_norm_bwd_scratch_elems.argtypes = [I, I]
    lib.b200_hstu_gate_cat_scratch_elems.argtypes = [I, I]
    lib.b200_hstu_gate_cat_scratch_elems.restype = c_ll
    lib.b200_norm_bwd_scratch_elems.restype = c_ll
    lib.b200_sumsq_scratch_elems.restype = c_int
    if hasattr(lib, "b200_sort_scratch_bytes"):
        lib.b200_sort_scratch_bytes.argtypes = [L]
        lib.b200_sort_scratch_bytes.restype = c_ll
    if hasattr(lib, "b200_segment_sum_scratch_elems"):
        lib.b200_segment_sum_scratch_elems.argtypes = [L, I]
        lib.b200_segment_sum_scratch_elems.restype = c_ll
    if hasattr(lib, "b200_gemm_grouped_mx_bn"):
        lib.b200_gemm_grouped_mx_bn.argtypes = [I]
        lib.b200_gemm_grouped_mx_bn.restype = c_int
    if hasattr(lib, "b200_zero_grid"):
        lib.b200_zero_grid.restype = c_int


def declare_extra(name: str, argtypes: list, restype=c_int) -> None:
    """Register the signature of a launcher added after this module was written."""
    lib = load()
    fn = getattr(lib, name)
    fn.argtypes = argtypes
    fn.restype = restype


def load() -> ctypes.CDLL:
    """Load the kernel library (once).  Raises RuntimeError with the reason on failure."""
    global _lib, _load_error
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if _load_error is not None:
            raise RuntimeError(_load_error)
        if not LIB_PATH.exists():
            _load_error = (f"{LIB_PATH} is missing: build it with "
                           f"`python -m mlperf_training_b200.csrc.build` (or __graft_entry__.build())")
            raise RuntimeError(_load_error)
        try:
            lib = ctypes.CDLL(str(LIB_PATH), mode=ctypes.RTLD_GLOBAL)
            _declare(lib)
        except (OSError, AttributeError) as e:  # pragma: no cover - depends on the machine
            _load_error = f"cannot load {LIB_PATH}: {e}"
            raise RuntimeError(_load_error) from e
        _lib = lib
        return lib


def available() -> bool:
    """True when CUDA is present and the kernel library loads."""
    if not torch.cuda.is_available():
        return False
    try:
        load()
        return True
    except RuntimeError:
        return False


def require() -> ctypes.CDLL:
    """The library, or a loud failure.  Called by every op that is handed a CUDA tensor."""
    return load()


def use_kernels(t: torch.Tensor) -> bool:
    """Dispatch rule of every op: CUDA tensors run the sm_100a kernels (and fail loudly when
    the library is absent); CPU tensors run the eager PyTorch definition of the same op."""
    if t.is_cuda:
        require()
        return True
    return False


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def call(name: str, *args) -> None:
    lib = load()
    rc = getattr(lib, name)(*args)
    if rc != 0:
        msg = lib.b200_last_error().decode(errors="replace")
        raise RuntimeError(f"{name} failed with code {rc}: {msg}")


def launch_count() -> int:
    return int(load().b200_launch_count()) if _lib is not None or LIB_PATH.exists() else 0


def reset_launch_count() -> None:
    load().b200_launch_count_reset()


def status() -> dict:
    """Read the device status block (synchronises).  ``code`` 0 means no kernel gave up a wait."""
    lib = load()
    buf = (c_int * 8)()
    rc = lib.b200_status_read(buf)
    if rc != 0:
        raise RuntimeError(lib.b200_last_error().decode(errors="replace"))
    return {"code": buf[0], "where": buf[1], "block": buf[2], "count": buf[3]}


def reset_status() -> None:
    lib = load()
    if lib.b200_status_reset() != 0:
        raise RuntimeError(lib.b200_last_error().decode(errors="replace"))


def check_status(what: str = "") -> None:
    st = status()
    if st["code"] != 0:
        reset_status()
        names = {1: "mbarrier wait timed out", 2: "flag wait timed out", 3: "bounds check failed"}
        raise RuntimeError(f"device status after {what or 'kernel'}: {names.get(st['code'], st['code'])} "
                           f"(where={st['where']}, block={st['block']}, reports={st['count']})")
