"""The validation source of a run: never the training files when a convergence target is set."""
import pytest

from mlperf_training_b200.parallel.mesh import MeshSpec, group_ranks
from mlperf_training_b200.trainer.loop import RunConfig, eval_spec


def test_synthetic_runs_draw_an_evaluation_stream_of_their_own():
    rc = RunConfig.from_dict({"data": {"kind": "synthetic", "loss_last": 8}, "eval_interval": 4, "target_eval_loss": 1.0})
    assert eval_spec(rc) == {"kind": "synthetic", "loss_last": 8}


def test_real_data_with_a_target_needs_validation_files():
    rc = RunConfig.from_dict({"data": {"kind": "indexed", "prefixes": ["/d/train"]}, "eval_interval": 4, "target_eval_loss": 3.3})
    with pytest.raises(ValueError, match="validation source"):
        eval_spec(rc)
    rc.data["valid_prefixes"] = ["/d/c4-validation"]
    assert eval_spec(rc)["prefixes"] == ["/d/c4-validation"]
    sft = RunConfig.from_dict({"data": {"kind": "packed_sft", "path": "/d/train.npy", "valid_path": "/d/validation.npy"},
                               "eval_interval": 48, "target_eval_loss": 0.925})
    assert eval_spec(sft)["path"] == "/d/validation.npy"
    explicit = RunConfig.from_dict({"data": {"kind": "packed_sft", "path": "/d/train.npy"},
                                    "eval_data": {"path": "/d/val.npy"}, "eval_interval": 48, "target_eval_loss": 0.925})
    assert eval_spec(explicit) == {"kind": "packed_sft", "path": "/d/val.npy"}


def test_expert_data_parallel_groups_hold_the_same_position_of_every_expert_block():
    g = group_ranks(MeshSpec(ep=2), 8)
    assert g["ep"] == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert g["edp"] == [[0, 2, 4, 6], [1, 3, 5, 7]]
