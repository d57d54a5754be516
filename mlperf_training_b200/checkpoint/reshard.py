"""Resume on a different number of data-parallel ranks than the checkpoint was written with.

A checkpoint directory holds one ``optim_rank<r>.pt`` per writer rank, each with the ``[lo, hi)`` slice of
every bucket's flat optimizer state (Adam moments, optional fp32 master weights).  The flat layout of a
bucket (parameter order and 8-element alignment) does not depend on the number of ranks, only its
padded length does, so a reader rank rebuilds its own slice by copying the overlaps out of the
writers' files.  The reference's fine-tuning run loads a ``torch_dist`` distributed checkpoint, whose
sharded tensors are likewise re-cut for whatever parallel layout reads them
(llama2_sft/primus/src/llama2_custom.py:711-725).
"""
from __future__ import annotations

import re
from pathlib import Path

import torch


def writer_files(ckpt_path) -> list[Path]:
    files = [f for f in Path(ckpt_path).glob("optim_rank*.pt") if re.fullmatch(r"optim_rank\d+\.pt", f.name)]
    return sorted(files, key=lambda f: int(re.findall(r"\d+", f.name)[0]))


def _copy_overlap(dst: torch.Tensor, dst_lo: int, src: torch.Tensor, src_lo: int, src_hi: int) -> int:
    a, z = max(dst_lo, src_lo), min(dst_lo + dst.numel(), src_hi)
    if a < z:
        dst[a - dst_lo:z - dst_lo].copy_(src[a - src_lo:z - src_lo])
    return max(z - a, 0)


def resharded_optimizer_state(ckpt_path, engine) -> dict:
    """``engine.load_optimizer_state`` input for ``engine``'s own sharding, assembled from every
    writer's file in ``ckpt_path``.  Buckets that are private to a rank (expert-parallel parameters) cannot
    be re-cut and raise."""
    files = writer_files(ckpt_path)
    if not files:
        raise FileNotFoundError(f"no optim_rank*.pt under {ckpt_path}")
    out = {"step": None, "buckets": {}}
    fresh = {}
    for b in engine.buckets:
        if getattr(b, "local_only", False):
            raise NotImplementedError(f"bucket {b.key} holds rank-private (expert-parallel) parameters: resume with the "
                                      "number of ranks the checkpoint was written with")
        fresh[b.key] = {"m": torch.zeros_like(b.m, device="cpu"), "v": torch.zeros_like(b.v, device="cpu"),
                        "master": None if b.master is None else torch.zeros_like(b.master, device="cpu"),
                        "lo": b.lo, "hi": b.hi, "names": [n for n, _ in b.params], "covered": 0}
    for f in files:
        old = torch.load(f, map_location="cpu", weights_only=False)
        out["step"] = int(old["step"]) if out["step"] is None else out["step"]
        for b in engine.buckets:
            ob, nb = old["buckets"].get(b.key), fresh[b.key]
            if ob is None:
                raise KeyError(f"{f.name} has no bucket '{b.key}'")
            if list(ob["names"]) != nb["names"]:
                raise ValueError(f"bucket '{b.key}': parameter list differs between checkpoint and model")
            lo, hi = int(ob["lo"]), int(ob["hi"])
            nb["covered"] += _copy_overlap(nb["m"], b.lo, ob["m"], lo, hi)
            _copy_overlap(nb["v"], b.lo, ob["v"], lo, hi)
            if nb["master"] is not None and ob.get("master") is not None:
                _copy_overlap(nb["master"], b.lo, ob["master"], lo, hi)
        del old
    for b in engine.buckets:
        nb = fresh[b.key]
        used = min(b.hi, _payload(b)) - min(b.lo, _payload(b))      # elements of this slice that hold parameters
        if nb.pop("covered") < used:
            raise ValueError(f"bucket '{b.key}': the checkpoint's files do not cover elements [{b.lo}, {b.hi})")
        out["buckets"][b.key] = nb
    return out


def _payload(b) -> int:
    """Elements of a bucket's flat buffer that belong to parameters (the rest is padding to the shard grid)."""
    n, p = b.params[-1]
    return b.offsets[-1] + p.numel()


def copy_param_bufs(engine, saved_bufs) -> None:
    """Full flat parameter buffers written under another padding: the common prefix carries the parameters."""
    for b, saved in zip(engine.buckets, saved_bufs):
        n = min(b.param_buf.numel(), saved.numel())
        if n < _payload(b):
            raise ValueError(f"bucket '{b.key}': saved buffer of {saved.numel()} elements is shorter than the parameters")
        b.param_buf[:n].copy_(saved[:n].to(b.param_buf.device))
