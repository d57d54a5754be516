"""Post-processing of exported Chrome traces (torch.profiler / Kineto JSON) into traces that load
cleanly and read correctly step by step.

An exported trace of a pipelined training run has four defects that make its timeline misleading:
GPU annotation spans that cross instead of nesting (clock skew between the activity buffers), kernel
slices of one stream that overlap by a few hundred nanoseconds, warm-up / lead-in work in front of the
first profiled step, and CPU annotations (``record_function`` / NVTX ranges) that have no GPU-side
span although their kernels ran later on the device.  The passes here repair each one:

* ``repair_gpu_nesting``     crossing GPU spans of one lane are made to nest (ends are moved, never starts);
* ``serialize_stream_order`` kernels / copies of one stream are put in launch order without overlap
                             (overlaps up to ``max_snap_us`` are snapped, larger ones reported);
* ``rename_lead_in_steps`` / ``clip_lead_in`` / ``trim_warmup``  the steps before the first complete
                             profiled step are labelled, clipped or dropped (with their flow events);
* ``rebuild_gpu_annotation_spans``  for every CPU annotation, the GPU span from the first to the last
                             kernel it launched (matched through correlation ids);
* ``step_wall_report``       per step: wall time, GPU busy time on the main stream, host self time,
                             exposed (non-overlapped) communication, and outlier steps.

``postprocess(path)`` runs them in order on a ``.json`` / ``.json.gz`` trace.  Same purpose as the
reference's trace tooling (generative_recommenders/dlrm_v4/trace_postprocessing.py: nesting repair
:44-219, stream serialisation :221-400, warm-up trimming :481-825, lead-in handling :836-861 and
:1466-1825, annotation rebuild :1097-1427, step report :947-1095, de-overlap :1827-1990).
"""
from __future__ import annotations

import gzip
import json
import re
import statistics
from pathlib import Path

GPU_CATS = ("kernel", "gpu_memcpy", "gpu_memset")
GPU_ANN = ("gpu_user_annotation",)
CPU_ANN = ("user_annotation", "cpu_op")
STEP_RE = re.compile(r"ProfilerStep#(\d+)|train_step[#_ ]?(\d+)|lead_in#(\d+)")


def load(path) -> dict:
    p = Path(path)
    raw = gzip.open(p, "rt").read() if p.suffix == ".gz" else p.read_text()
    data = json.loads(raw)
    return data if isinstance(data, dict) else {"traceEvents": data}


def save(data: dict, path) -> None:
    p = Path(path)
    raw = json.dumps(data)
    if p.suffix == ".gz":
        with gzip.open(p, "wt") as f:
            f.write(raw)
    else:
        p.write_text(raw)


def _x(events, cats=None):
    return [e for e in events if e.get("ph") == "X" and (cats is None or e.get("cat") in cats)]


def _end(e) -> float:
    return e["ts"] + e.get("dur", 0)


def _lanes(evts):
    lanes: dict = {}
    for e in evts:
        lanes.setdefault((e.get("pid"), e.get("tid")), []).append(e)
    return lanes


# ----------------------------------------------------------------------------------------------
def repair_gpu_nesting(events: list) -> int:
    """Spans of one lane must be disjoint or nested.  A span that starts inside another and ends after it
    is shortened to end with its parent; returns the number of ends moved."""
    moved = 0
    for lane in _lanes(_x(events, GPU_ANN)).values():
        lane.sort(key=lambda e: (e["ts"], -e.get("dur", 0)))
        stack: list = []
        for e in lane:
            while stack and _end(stack[-1]) <= e["ts"]:
                stack.pop()
            if stack and _end(e) > _end(stack[-1]):
                e["dur"] = max(_end(stack[-1]) - e["ts"], 0)
                e.setdefault("args", {})["nesting_repaired"] = True
                moved += 1
            stack.append(e)
    return moved


def serialize_stream_order(events: list, max_snap_us: float = 5.0) -> dict:
    """Device work of one stream executes in order: every slice starts at or after the end of the previous
    one.  Overlaps up to ``max_snap_us`` are timestamp noise and are snapped; larger ones are kept in order
    (start moved, duration reduced) and counted as ``large``."""
    stats = {"snapped": 0, "large": 0}
    for lane in _lanes(_x(events, GPU_CATS)).values():
        lane.sort(key=lambda e: e["ts"])
        end = None
        for e in lane:
            if end is not None and e["ts"] < end:
                shift = end - e["ts"]
                stats["snapped" if shift <= max_snap_us else "large"] += 1
                e["dur"] = max(e.get("dur", 0) - shift, 0)
                e["ts"] = end
            end = _end(e)
    return stats


# ----------------------------------------------------------------------------------------------
def step_spans(events: list) -> list:
    """(step number, event) of the CPU-side step ranges, in time order."""
    out = []
    for e in _x(events):
        m = STEP_RE.search(str(e.get("name", "")))
        if m and e.get("cat") not in GPU_CATS + GPU_ANN:
            out.append((int(m.group(1) or m.group(2) or m.group(3)), e))
    return sorted(out, key=lambda t: t[1]["ts"])


def rename_lead_in_steps(events: list, first_timed: int | None = None) -> int:
    """Step ranges before the first timed step are lead-in (warm-up inside the profiler window): rename
    them so the step report and a reader skip them.  ``first_timed`` defaults to the second recorded step
    (the first one carries the profiler's own start-up)."""
    spans = step_spans(events)
    if not spans:
        return 0
    numbers = sorted({n for n, _ in spans})
    cut = first_timed if first_timed is not None else (numbers[1] if len(numbers) > 1 else numbers[0])
    n = 0
    for num, e in spans:
        if num < cut:
            e["name"] = f"lead_in#{num}"
            n += 1
    return n


def trim_warmup(data: dict, before_us: float) -> dict:
    """Drop every event that ends before ``before_us`` and clip those that straddle it; flow events whose
    partner was dropped go too.  Returns counters."""
    events = data["traceEvents"]
    stats = {"dropped": 0, "clipped": 0, "flows_dropped": 0}
    keep, dropped_ids = [], set()
    for e in events:
        if e.get("ph") == "X":
            if _end(e) <= before_us:
                stats["dropped"] += 1
                if "args" in e and "correlation" in e["args"]:
                    dropped_ids.add(e["args"]["correlation"])
                continue
            if e["ts"] < before_us:
                e["dur"] = _end(e) - before_us
                e["ts"] = before_us
                stats["clipped"] += 1
        keep.append(e)
    out = []
    for e in keep:
        if e.get("ph") in ("s", "f", "t") and (e.get("ts", before_us) < before_us or e.get("id") in dropped_ids):
            stats["flows_dropped"] += 1
            continue
        out.append(e)
    data["traceEvents"] = out
    return stats


def clip_lead_in(data: dict) -> dict:
    """Trim the trace at the start of the first step that is not a lead-in step."""
    timed = [e for _, e in step_spans(data["traceEvents"]) if not str(e["name"]).startswith("lead_in#")]
    if not timed:
        return {"dropped": 0, "clipped": 0, "flows_dropped": 0}
    return trim_warmup(data, timed[0]["ts"])


# ----------------------------------------------------------------------------------------------
def rebuild_gpu_annotation_spans(events: list, gpu_pid=None) -> int:
    """For every CPU annotation, add a GPU-side span from the start of the first to the end of the last
    kernel launched inside it (kernels are tied to their launch calls by ``args.correlation``).  Returns
    the number of spans added."""
    launches = [e for e in _x(events, ("cuda_runtime", "cuda_driver")) if "correlation" in e.get("args", {})]
    kernels = {}
    for k in _x(events, GPU_CATS):
        c = k.get("args", {}).get("correlation")
        if c is not None:
            kernels[c] = k
    launches.sort(key=lambda e: e["ts"])
    added = 0
    for a in _x(events, ("user_annotation",)):
        lo, hi = a["ts"], _end(a)
        ks = [kernels[l["args"]["correlation"]] for l in launches
              if l.get("pid") == a.get("pid") and l.get("tid") == a.get("tid") and lo <= l["ts"] < hi
              and l["args"]["correlation"] in kernels]
        if not ks:
            continue
        t0, t1 = min(k["ts"] for k in ks), max(_end(k) for k in ks)
        events.append({"ph": "X", "cat": "gpu_user_annotation", "name": a["name"], "ts": t0, "dur": t1 - t0,
                       "pid": gpu_pid if gpu_pid is not None else ks[0].get("pid"), "tid": ks[0].get("tid"),
                       "args": {"rebuilt_from_cpu": True, "kernels": len(ks)}})
        added += 1
    return added


# ----------------------------------------------------------------------------------------------
def _busy(slices, lo, hi) -> float:
    """Union length of the slices inside [lo, hi]."""
    iv = sorted((max(s["ts"], lo), min(_end(s), hi)) for s in slices if s["ts"] < hi and _end(s) > lo)
    tot, cur_lo, cur_hi = 0.0, None, None
    for a, b in iv:
        if cur_hi is None or a > cur_hi:
            if cur_hi is not None:
                tot += cur_hi - cur_lo
            cur_lo, cur_hi = a, b
        else:
            cur_hi = max(cur_hi, b)
    if cur_hi is not None:
        tot += cur_hi - cur_lo
    return tot


def step_wall_report(events: list, comm_pattern: str = r"nccl|all_gather|reduce_scatter|mc_all_gather|zero_reduce") -> dict:
    """Per timed step: wall, GPU busy on the busiest stream ("main"), busy on all streams, exposed
    communication (communication kernels not covered by other device work), host self time of the step's
    thread; plus the median wall and the steps that are more than 25 % away from it."""
    kernels = _x(events, GPU_CATS)
    lanes = _lanes(kernels)
    main = max(lanes.values(), key=lambda l: sum(e.get("dur", 0) for e in l)) if lanes else []
    comm_re = re.compile(comm_pattern, re.I)
    comm = [k for k in kernels if comm_re.search(str(k.get("name", "")))]
    compute = [k for k in kernels if not comm_re.search(str(k.get("name", "")))]
    rows = []
    for num, s in step_spans(events):
        if str(s["name"]).startswith("lead_in#"):
            continue
        lo, hi = s["ts"], _end(s)
        cpu_children = [e for e in _x(events, CPU_ANN + ("cuda_runtime",)) if e.get("pid") == s.get("pid")
                        and e.get("tid") == s.get("tid") and e is not s and lo <= e["ts"] and _end(e) <= hi]
        exposed = _busy(comm, lo, hi) - (_busy(comm, lo, hi) + _busy(compute, lo, hi) - _busy(comm + compute, lo, hi))
        rows.append({"step": num, "wall_us": hi - lo, "gpu_main_busy_us": _busy(main, lo, hi),
                     "gpu_busy_us": _busy(kernels, lo, hi), "exposed_comm_us": max(exposed, 0.0),
                     "host_self_us": (hi - lo) - _busy(cpu_children, lo, hi)})
    walls = [r["wall_us"] for r in rows]
    med = statistics.median(walls) if walls else 0.0
    return {"steps": rows, "median_wall_us": med,
            "outliers": [r["step"] for r in rows if med and abs(r["wall_us"] - med) > 0.25 * med]}


def postprocess(path, out=None, drop_lead_in: bool = True, max_snap_us: float = 5.0) -> dict:
    """All passes on one trace file; writes ``out`` (default: in place) and returns the counters and the
    step report."""
    data = load(path)
    ev = data["traceEvents"]
    stats = {"lead_in_steps": rename_lead_in_steps(ev)}
    if drop_lead_in:
        stats["trim"] = clip_lead_in(data)
        ev = data["traceEvents"]
    stats["stream_order"] = serialize_stream_order(ev, max_snap_us)
    stats["annotations_rebuilt"] = rebuild_gpu_annotation_spans(ev)
    stats["nesting_moved"] = repair_gpu_nesting(ev)
    stats["report"] = step_wall_report(ev)
    save(data, out or path)
    return stats


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(description="repair and summarise an exported Chrome trace")
    ap.add_argument("trace")
    ap.add_argument("--out", default=None)
    ap.add_argument("--keep-lead-in", action="store_true")
    args = ap.parse_args(argv)
    stats = postprocess(args.trace, args.out, drop_lead_in=not args.keep_lead_in)
    rep = stats.pop("report")
    print(json.dumps(stats))
    print(json.dumps({k: rep[k] for k in ("median_wall_us", "outliers")}))
    for r in rep["steps"]:
        print(json.dumps(r))
    return 0


if __name__ == "__main__":
    import sys
    sys.exit(main())
