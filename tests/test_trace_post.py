"""Trace post-processing passes on a hand-made Chrome trace."""
import json

from mlperf_training_b200.utils import trace_post as T


def _trace():
    ev = []
    # three CPU step ranges on pid 1 / tid 1; kernels on GPU pid 0, streams 7 (compute) and 9 (comm)
    for n, t0 in ((3, 0), (4, 1000), (5, 2000)):
        ev.append({"ph": "X", "cat": "user_annotation", "name": f"ProfilerStep#{n}", "ts": t0, "dur": 1000, "pid": 1, "tid": 1})
        ev.append({"ph": "X", "cat": "user_annotation", "name": "fwd", "ts": t0 + 10, "dur": 300, "pid": 1, "tid": 1})
        for j in range(3):
            c = n * 10 + j
            ev.append({"ph": "X", "cat": "cuda_runtime", "name": "cudaLaunchKernel", "ts": t0 + 20 + 50 * j, "dur": 5, "pid": 1, "tid": 1,
                       "args": {"correlation": c}})
            ev.append({"ph": "X", "cat": "kernel", "name": f"gemm_pair_kernel_{j}", "ts": t0 + 100 + 200 * j, "dur": 202, "pid": 0, "tid": 7,
                       "args": {"correlation": c}})                                     # 2 us overlap with the next one
            ev.append({"ph": "s", "id": c, "ts": t0 + 20 + 50 * j, "pid": 1, "tid": 1, "cat": "ac2g", "name": "ac2g"})
        ev.append({"ph": "X", "cat": "kernel", "name": "ncclDevKernel_AllGather", "ts": t0 + 600, "dur": 300, "pid": 0, "tid": 9,
                   "args": {"correlation": n * 10 + 9}})
    # crossing GPU annotation spans on one lane
    ev.append({"ph": "X", "cat": "gpu_user_annotation", "name": "outer", "ts": 2100, "dur": 400, "pid": 0, "tid": 7})
    ev.append({"ph": "X", "cat": "gpu_user_annotation", "name": "inner", "ts": 2300, "dur": 400, "pid": 0, "tid": 7})
    return {"traceEvents": ev}


def test_passes(tmp_path):
    data = _trace()
    ev = data["traceEvents"]
    assert T.rename_lead_in_steps(ev) == 1                                   # step 3 is lead-in
    assert [e["name"] for _, e in T.step_spans(ev)][0] == "lead_in#3"
    trim = T.clip_lead_in(data)
    ev = data["traceEvents"]
    assert trim["dropped"] > 0 and min(e["ts"] for e in ev if e.get("ph") == "X") >= 1000
    assert all(e.get("ts", 1000) >= 1000 for e in ev if e.get("ph") == "s")
    so = T.serialize_stream_order(ev)
    assert so["snapped"] == 4 and so["large"] == 0
    lane = sorted((e for e in ev if e.get("cat") == "kernel" and e["tid"] == 7), key=lambda e: e["ts"])
    assert all(a["ts"] + a["dur"] <= b["ts"] for a, b in zip(lane, lane[1:]))
    added = T.rebuild_gpu_annotation_spans(ev)
    assert added >= 2
    fwd = [e for e in ev if e.get("cat") == "gpu_user_annotation" and e["name"] == "fwd"]
    assert fwd and fwd[0]["args"]["kernels"] == 3 and fwd[0]["ts"] == 1100
    assert T.repair_gpu_nesting(ev) >= 1
    inner = next(e for e in ev if e.get("name") == "inner")
    assert inner["ts"] + inner["dur"] == 2500
    rep = T.step_wall_report(ev)
    assert [r["step"] for r in rep["steps"]] == [4, 5] and rep["median_wall_us"] == 1000
    r = rep["steps"][0]
    assert abs(r["gpu_main_busy_us"] - 602) < 1e-6 and 0 < r["exposed_comm_us"] <= 300 and r["host_self_us"] < 1000
    p = tmp_path / "t.json.gz"
    T.save(_trace(), p)
    stats = T.postprocess(p)
    assert stats["lead_in_steps"] == 1 and json.dumps(stats)
    assert T.load(p)["traceEvents"]


def test_run_loop_trace_carries_step_ranges(tmp_path):
    """A trace recorded by the run loop (``profile_step_start`` / ``profile_step_end``) marks every profiled step, so the
    post-processing finds the steps it reports on."""
    import glob
    import io

    from mlperf_training_b200.trainer.loop import run
    from mlperf_training_b200.utils.trace_post import postprocess
    tiny = dict(n_layers=1, hidden=32, n_heads=2, n_kv_heads=1, head_dim=16, ffn_hidden=64, vocab_size=64, seq_len=16, dtype="fp32")
    run(dict(model=tiny, global_batch=2, micro_batch=1, train_iters=5, profile_step_start=1, profile_step_end=4,
             profile_dir=str(tmp_path)), device="cpu", stream=io.StringIO())
    rep = postprocess(glob.glob(str(tmp_path / "trace_rank0.json*"))[0], out=str(tmp_path / "fixed.json"), drop_lead_in=False)
    steps = [s["step"] for s in rep["report"]["steps"]]
    assert steps and set(steps) <= {1, 2, 3} and rep["report"]["median_wall_us"] > 0


def test_hstu_loop_trace_carries_step_ranges(tmp_path):
    import glob
    import io

    from mlperf_training_b200.trainer.hstu import run
    from mlperf_training_b200.utils.trace_post import postprocess
    e = dict(batch_per_gpu=4, train_steps=5, eval_interval_steps=0, num_eval_batches=0, profile_step_start=1, profile_step_end=4,
             profile_dir=str(tmp_path),
             model=dict(layers=1, dim=32, heads=2, d_qk=16, d_v=16, max_seq_len=48, dtype="fp32", mlp_hidden=16, num_positions=64,
                        num_time_buckets=32),
             embedding=dict(rows=200, dim=16), data=dict(length_median=12, length_min=4, length_max=40))
    run(e, device="cpu", stream=io.StringIO())
    rep = postprocess(glob.glob(str(tmp_path / "trace_rank0.json*"))[0], out=str(tmp_path / "fixed.json"), drop_lead_in=False)
    assert [s["step"] for s in rep["report"]["steps"]] == [2, 3]          # the first profiled step is the lead-in
