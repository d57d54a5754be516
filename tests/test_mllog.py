"""MLLOG logger: submission metadata."""


def test_submission_metadata_comes_from_the_environment(monkeypatch):
    import io
    import json
    from mlperf_training_b200.mllog import core as ml
    monkeypatch.setenv("MLLOG_SUBMISSION_PLATFORM", "1xB200_test")
    out = io.StringIO()
    log = ml.MLLogger(rank=0, stream=out)
    log.log_submission("llama31_8b")
    recs = [json.loads(l.split(":::MLLOG", 1)[1]) for l in out.getvalue().splitlines() if ":::MLLOG" in l]
    vals = {r["key"]: r["value"] for r in recs}
    assert vals["submission_platform"] == "1xB200_test" and vals["submission_benchmark"] == "llama31_8b"
