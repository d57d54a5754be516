"""Sort / unique / segment-sum of the sparse path.

``sort_unique(ids, key_bits)`` -> ``SortedIds``: ids sorted (stable) with each one's original
position, the unique ids, run offsets, the number of runs (a device scalar: no host read) and the
inverse map.  ``segment_sum(src, s, out_dtype)`` sums the rows of ``src`` that carry the same id in
sorted (fixed) order.  CUDA tensors run the kernels of csrc/sort.cu (bounded-key radix sort); CPU
tensors run ``torch.sort(stable=True)`` + run arithmetic - the oracle of the GPU tests.

Counterparts in the reference: the bounded-key onesweep radix sort
(generative_recommenders/ops/onesweep_sort_kernels.hip:39-110) and the deterministic segment
reduction of duplicate embedding gradients (generative_recommenders/dlrm_v4/train/ec_segment_reduce.py).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ._lib import call, load, ptr, stream_ptr, use_kernels


@dataclass
class SortedIds:
    keys: torch.Tensor        # [n] sorted ids
    perm: torch.Tensor        # [n] original position of every sorted id
    uniq: torch.Tensor        # [n] (first ``count`` entries valid) unique ids, ascending
    seg: torch.Tensor         # [n + 1] (first ``count + 1`` valid) start of every run in ``keys``
    inverse: torch.Tensor     # [n] run index of every ORIGINAL position
    count: torch.Tensor       # [1] number of runs, on the device

    def n_unique(self) -> int:
        """Host read of the run count (synchronises; the kernels never need it)."""
        return int(self.count.item())


def key_bits_for(rows: int) -> int:
    """Bits a radix sort has to look at for ids in ``[0, rows)``."""
    return max(int(rows - 1).bit_length(), 1)


_scratch: dict = {}


def _scratch_for(n: int, device) -> torch.Tensor:
    need = int(load().b200_sort_scratch_bytes(n))
    buf = _scratch.get(device)
    if buf is None or buf.numel() < need:
        buf = _scratch[device] = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=device)
    return buf


def sort_unique(ids: torch.Tensor, key_bits: int = 64) -> SortedIds:
    ids = ids.reshape(-1).to(torch.int64)
    n = ids.numel()
    dev = ids.device
    if not use_kernels(ids):
        keys, perm = torch.sort(ids, stable=True)
        head = torch.ones(n, dtype=torch.bool)
        head[1:] = keys[1:] != keys[:-1]
        run = torch.cumsum(head.long(), 0) - 1
        cnt = int(run[-1]) + 1 if n else 0
        uniq = torch.full((n,), -1, dtype=torch.int64)
        seg = torch.zeros(n + 1, dtype=torch.int64)
        uniq[:cnt] = keys[head]
        seg[:cnt] = torch.nonzero(head)[:, 0]
        seg[cnt] = n
        inverse = torch.empty(n, dtype=torch.int64)
        inverse[perm] = run
        return SortedIds(keys, perm, uniq, seg, inverse, torch.tensor([cnt]))
    keys = torch.empty_like(ids)
    perm = torch.empty_like(ids)
    uniq = torch.full_like(ids, -1)              # entries past the run count stay -1 (consumers skip them)
    seg = torch.empty(n + 1, dtype=torch.int64, device=dev)
    inverse = torch.empty_like(ids)
    count = torch.zeros(1, dtype=torch.int64, device=dev)
    if n:
        scratch = _scratch_for(n, dev)
        call("b200_sort_ids", ptr(ids.contiguous()), ptr(keys), ptr(perm), n, int(min(max(key_bits, 1), 64)), ptr(scratch),
             scratch.numel(), stream_ptr())
        call("b200_unique_segments", ptr(keys), ptr(perm), n, ptr(uniq), ptr(seg), ptr(inverse), ptr(count), ptr(scratch),
             scratch.numel(), stream_ptr())
    return SortedIds(keys, perm, uniq, seg, inverse, count)


def segment_sum(src: torch.Tensor, s: SortedIds, out_dtype=torch.float32, max_seg: int | None = None) -> torch.Tensor:
    """``out[j] = sum of src[p] over the original positions p whose id is the j-th unique id`` (sorted
    order inside a run).  Returns ``[n, D]`` rows (the first ``count`` are valid; the rest untouched zeros)."""
    n, D = s.keys.numel(), src.shape[1]
    out = torch.zeros((n if max_seg is None else max_seg, D), dtype=out_dtype, device=src.device)
    if n == 0:
        return out
    if not use_kernels(src):
        cnt = int(s.count)
        acc = torch.zeros((cnt, D), dtype=torch.float32)
        acc.index_add_(0, s.inverse, src.float())      # CPU index_add_ runs in index order: deterministic
        out[:cnt] = acc.to(out_dtype)
        return out
    if src.dtype not in (torch.bfloat16, torch.float32) or out_dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("segment_sum: bf16 or fp32 rows")
    from . import _lib
    # partial sums of the runs that are too long for one warp (skewed ids): one fp32 row pair per 64 sorted positions
    partial = torch.empty(int(_lib.load().b200_segment_sum_scratch_elems(n, D)), dtype=torch.float32, device=src.device)
    call("b200_segment_sum_gather", ptr(src.contiguous()), int(src.dtype == torch.float32), src.shape[0], ptr(s.perm), ptr(s.seg), ptr(s.count),
         n, out.shape[0], D, ptr(out), int(out_dtype == torch.bfloat16), ptr(partial), stream_ptr())
    return out
