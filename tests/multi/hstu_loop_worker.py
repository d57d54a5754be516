"""Worker (gloo, 2 ranks): the HSTU run loop over the eleven-table feature set with two tables cut along their width,
the rest placed by the planner; a run that exits after a sharded sparse checkpoint resumes onto the straight run's
losses.  argv: <checkpoint root>"""
import io
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.parallel.embedding import ColumnShardedEmbedding  # noqa: E402
from mlperf_training_b200.trainer.hstu import run  # noqa: E402


def exp(**over):
    e = dict(batch_per_gpu=4, train_steps=8, dense_lr=2e-3, sparse_lr=0.05, eval_interval_steps=0, num_eval_batches=0,
             model=dict(layers=2, dim=32, heads=2, d_qk=16, d_v=16, max_seq_len=64, dtype="fp32", mlp_hidden=32, num_positions=256,
                        num_time_buckets=64, input_dropout=0.0, linear_dropout=0.0),
             embedding=dict(rows=200, dim=16, tables="yambda", table_scale=20000, column_wise=["item_id", "uid"]),
             data=dict(length_median=12, length_min=4, length_max=40))
    e.update(over)
    return e


def main():
    root = sys.argv[1]
    rank = int(os.environ["RANK"])
    dist.init_process_group("gloo")
    ref = run(exp(), device="cpu", stream=io.StringIO())
    tabs = ref["trainer"].table.tables
    ok = isinstance(tabs["item_id"], ColumnShardedEmbedding) and tabs["item_id"].weight.shape[1] == 8
    ok &= not isinstance(tabs["cross_0"], ColumnShardedEmbedding)
    ok &= all(l == l for l in ref["losses"]) and len(ref["losses"]) == 8
    e = exp(checkpoint_dir=os.path.join(root, "ck"), die_at_step=4, sparse_checkpoint="sharded")
    try:
        run(dict(e), device="cpu", stream=io.StringIO())
        ok = False
    except SystemExit as ex:
        ok &= int(ex.code) == 42
    out = run(dict(e, die_at_step=0), device="cpu", stream=io.StringIO())
    ok &= len(out["losses"]) == 4 and max(abs(a - b) for a, b in zip(out["losses"], ref["losses"][4:])) < 1e-5
    t = torch.tensor(out["losses"], dtype=torch.float64)
    print(f"RESULT rank {rank} ok={bool(ok)} last {float(t[-1]):.6f} ref {ref['losses'][-1]:.6f}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
