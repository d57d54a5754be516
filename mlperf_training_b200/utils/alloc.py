"""Caching-allocator control for steady-state steps.

``pregrow`` reserves device memory up front (on the streams a pipeline will use) so the allocator
never has to map new segments after the run has started; ``GrowthMonitor`` reports any growth that
still happens, step by step.  The reference does this for the same reason - a ``cudaMalloc`` in the
timed region synchronises the device and fragments the heap
(generative_recommenders/dlrm_v4/alloc_pregrow.py:1-498: pre-mapped per-stream expandable segments
and a growth reporter; generative_recommenders/ops/triton/fp8_tm_alloc.py: a private pool for the
token-major FP8 operands).
"""
from __future__ import annotations

import torch


def recommended_env() -> dict:
    """Allocator settings the launch scripts export (expandable segments avoid fragmentation when
    jagged batches change size every step)."""
    return {"PYTORCH_CUDA_ALLOC_CONF": "expandable_segments:True"}


def pregrow(bytes_per_stream: int, streams=None, device=None) -> int:
    """Allocate and release ``bytes_per_stream`` on every stream so the blocks stay cached for them.
    Returns the bytes reserved afterwards (0 on CPU)."""
    if not torch.cuda.is_available():
        return 0
    device = device if device is not None else torch.cuda.current_device()
    streams = streams or [torch.cuda.current_stream(device)]
    for s in streams:
        with torch.cuda.stream(s):
            block = torch.empty(bytes_per_stream, dtype=torch.uint8, device=device)
            del block
    torch.cuda.synchronize(device)
    return int(torch.cuda.memory_reserved(device))


class PrivatePool:
    """A separate allocator pool for tensors with a different lifetime pattern (e.g. quantised
    operands that live across forward and backward), so they do not fragment the main pool."""

    def __init__(self, device=None):
        self.enabled = torch.cuda.is_available()
        self.pool = torch.cuda.graph_pool_handle() if self.enabled else None
        self.device = device
        self._ctx = None

    def __enter__(self):
        if self.enabled and hasattr(torch.cuda, "use_mem_pool") and hasattr(torch.cuda, "MemPool"):
            self._mem = getattr(self, "_mem", None) or torch.cuda.MemPool()
            self._ctx = torch.cuda.use_mem_pool(self._mem)
            self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        if self._ctx is not None:
            self._ctx.__exit__(*exc)
            self._ctx = None
        return False


class GrowthMonitor:
    def __init__(self, device=None, stats=None):
        self._stats = stats or (lambda: torch.cuda.memory_stats(device) if torch.cuda.is_available() else {})
        self.base = self._snapshot()
        self.events: list[dict] = []

    def _snapshot(self) -> dict:
        s = self._stats()
        return {"reserved": int(s.get("reserved_bytes.all.current", 0)), "segments": int(s.get("segment.all.allocated", 0)),
                "retries": int(s.get("num_alloc_retries", 0))}

    def check(self, step: int) -> dict | None:
        now = self._snapshot()
        grew = {k: now[k] - self.base[k] for k in now if now[k] > self.base[k]}
        self.base = now
        if grew:
            ev = {"step": step, **grew}
            self.events.append(ev)
            return ev
        return None

    def report(self) -> str:
        if not self.events:
            return "allocator: no growth after start"
        tot = sum(e.get("reserved", 0) for e in self.events)
        return f"allocator: grew {len(self.events)} time(s), +{tot / 2**20:.1f} MiB reserved (first at step {self.events[0]['step']})"
