"""Step-window profiling: a ``torch.profiler`` wrapper with a rank-aligned start, NVTX step ranges
and a Chrome-trace export, plus the device-time helpers the benchmarks use.

The reference wraps ``torch.profiler`` the same way (single or multi-window schedule, rank-aligned
start behind a barrier, on-trace-ready export followed by a trace clean-up pass:
generative_recommenders/dlrm_v4/utils.py:451-822, YAML knobs ``profile_step_start/end`` in
small_llm_pretraining/primus/conf/llama3.1_8B-pretrain-fp4.yaml:76-84).
"""
from __future__ import annotations

import contextlib
import gzip
import json
import os
import shutil
from pathlib import Path

import torch


class StepProfiler:
    def __init__(self, out_dir: str, rank: int = 0, gzip_trace: bool = True, with_cpu: bool = True):
        self.out_dir = Path(out_dir)
        self.rank = rank
        self.gzip = gzip_trace
        acts = [torch.profiler.ProfilerActivity.CPU] if with_cpu else []
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self.prof = torch.profiler.profile(activities=acts, record_shapes=False)
        self.path: Path | None = None

    def start(self) -> None:
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            torch.distributed.barrier()
        self.prof.start()

    def step_range(self, step: int):
        """Context manager that marks one training step in the trace (``train_step#<n>``): the ranges the trace
        post-processing cuts the timeline by (``utils.trace_post.step_spans``)."""
        return torch.profiler.record_function(f"train_step#{int(step)}")

    def stop(self) -> Path:
        self.prof.stop()
        self.out_dir.mkdir(parents=True, exist_ok=True)
        p = self.out_dir / f"trace_rank{self.rank}.json"
        self.prof.export_chrome_trace(str(p))
        clean_trace(p)
        if self.gzip:
            with open(p, "rb") as src, gzip.open(str(p) + ".gz", "wb") as dst:
                shutil.copyfileobj(src, dst)
            p.unlink()
            p = Path(str(p) + ".gz")
        self.path = p
        return p


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range around a region when CUDA is present (shows up in nsys / ncu timelines)."""
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


def clean_trace(path: str | os.PathLike, trim_before_us: float | None = None) -> dict:
    """Post-process a Chrome trace in place: drop events that start before ``trim_before_us``
    (warm-up lead-in), clip negative durations, and serialise events that overlap on the same
    (pid, tid) lane so every lane is a valid nesting - the repairs the reference applies to its
    exported traces (generative_recommenders/dlrm_v4/trace_postprocessing.py).  Returns counters."""
    path = Path(path)
    data = json.loads(path.read_text())
    events = data.get("traceEvents", data if isinstance(data, list) else [])
    stats = {"dropped": 0, "clipped": 0, "deoverlapped": 0}
    keep = []
    for e in events:
        if e.get("ph") == "X":
            if trim_before_us is not None and e.get("ts", 0) < trim_before_us:
                stats["dropped"] += 1
                continue
            if e.get("dur", 0) < 0:
                e["dur"] = 0
                stats["clipped"] += 1
        keep.append(e)
    lanes: dict = {}
    for e in keep:
        if e.get("ph") == "X" and e.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset"):
            lanes.setdefault((e.get("pid"), e.get("tid")), []).append(e)
    for lane in lanes.values():
        lane.sort(key=lambda e: e["ts"])
        end = None
        for e in lane:
            if end is not None and e["ts"] < end:
                shift = end - e["ts"]
                e["dur"] = max(e.get("dur", 0) - shift, 0)
                e["ts"] = end
                stats["deoverlapped"] += 1
            end = e["ts"] + e.get("dur", 0)
    if isinstance(data, dict):
        data["traceEvents"] = keep
        path.write_text(json.dumps(data))
    else:
        path.write_text(json.dumps(keep))
    return stats


def step_wall_report(path: str | os.PathLike, marker: str = "train_step") -> dict:
    """Per-step wall and GPU-busy time from a trace that contains ``marker`` ranges."""
    p = Path(path)
    raw = gzip.open(p, "rt").read() if p.suffix == ".gz" else p.read_text()
    data = json.loads(raw)
    events = data.get("traceEvents", [])
    steps = sorted((e for e in events if e.get("ph") == "X" and marker in str(e.get("name", ""))), key=lambda e: e["ts"])
    kernels = [e for e in events if e.get("ph") == "X" and e.get("cat") == "kernel"]
    out = []
    for s in steps:
        lo, hi = s["ts"], s["ts"] + s.get("dur", 0)
        busy = sum(min(k["ts"] + k.get("dur", 0), hi) - max(k["ts"], lo) for k in kernels
                   if k["ts"] < hi and k["ts"] + k.get("dur", 0) > lo)
        out.append({"wall_us": s.get("dur", 0), "gpu_busy_us": busy})
    return {"steps": out}


# peak dense bf16 TFLOP/s used for MFU lines (generative_recommenders/dlrm_v4/utils.py:1634-1648)
GPU_PEAK_TFLOPS = {"B200": 2250.0, "H100": 990.0, "H200": 990.0, "A100": 312.0, "MI355X": 2500.0, "MI350X": 2300.0}


def gpu_peak_tflops(name: str | None = None) -> float:
    if name is None and torch.cuda.is_available():
        name = torch.cuda.get_device_name()
    for k, v in GPU_PEAK_TFLOPS.items():
        if name and k in name:
            return v
    return 0.0
